"""Video classification in the UCF101 layout: per-frame ResNet features -> 2-layer LSTM -> mean over time.

    python samples/ucf101_resnetlstm.py [--data-dir DIR] [--resnet-size 50] [--epochs 1] [--mode majority]

The reference's sample of the same name (deep500 samples/ucf101_resnetlstm.py:18-113): ResNet-50 features of
every frame, an LSTM with hidden size 256 and dropout 0.5, a fully connected layer and the time mean of its
outputs; batches of 4 clips drawn from length buckets (``BucketSampler``, at most 500 frames, 30 buckets),
clips left-padded and sub-sampled by the loader.  Without ``--data-dir`` a small synthetic data set in the
UCF101 layout is written to a temporary directory first.  Clips of different length make ranks finish their
steps at different times: the load imbalance eager-SGD was made for.
"""
import argparse
import os
import sys
import tempfile
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import eagersgd_b200 as es  # noqa: E402
from eagersgd_b200.data import BucketSampler, VideoFolderDataset, VideoLoader, write_synthetic_ucf101  # noqa: E402
from eagersgd_b200.models.resnet import cifar_resnet  # noqa: E402
from eagersgd_b200.models.video import ResNetLSTM  # noqa: E402
from eagersgd_b200.ops.functional import softmax_cross_entropy  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--data-dir", default=None, help="UCF101-style directory of decoded clips (.npy) and list files")
    ap.add_argument("--mode", default="majority", choices=["solo", "majority", "sync"])
    ap.add_argument("--resnet-size", type=int, default=50, help="ImageNet ResNet depth of the frame network; "
                    "8 .. 56 selects a CIFAR-style one (small frames)")
    ap.add_argument("--hidden", type=int, default=256)
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--epochs", type=int, default=1)
    ap.add_argument("--max-length", type=int, default=500)
    ap.add_argument("--skip-frames", type=int, default=10)
    ap.add_argument("--max-steps", type=int, default=0)
    args = ap.parse_args()
    group = es.init()
    dev = group.device
    torch.manual_seed(0)
    root = args.data_dir or write_synthetic_ucf101(os.path.join(tempfile.mkdtemp(), "ucf101"), classes=4, seed=1)
    loader = VideoLoader(normalize=True, max_length=args.max_length * args.skip_frames, skip_frames=args.skip_frames)
    train = VideoFolderDataset(root, "trainlist01.txt", loader)
    classes = len(train.classes)
    if args.resnet_size < 18:
        frame_net = cifar_resnet(args.resnet_size, 1, 10)
        model = ResNetLSTM(classes, hidden=args.hidden, frame_net=frame_net, feature_dim=frame_net.fc.in_features)
    else:
        model = ResNetLSTM(classes, resnet_size=args.resnet_size, hidden=args.hidden)
    model = model.to(dev)
    if dev.type == "cuda":
        from eagersgd_b200.train.step import prepare_model
        model = prepare_model(model, dev)
    sampler = BucketSampler(train, args.batch, train.lengths, num_buckets=30, max_length=args.max_length,
                            seed=group.rank)
    inner = torch.optim.SGD(model.parameters(), lr=0.01, momentum=0.9)
    cls = {"solo": es.SoloAllreduceOptimizer, "majority": es.MajorityAllreduceOptimizer, "sync": es.SyncAllreduceOptimizer}
    opt = cls[args.mode](inner, group)
    clips, steps, t0, loss = 0, 0, time.time(), None
    for epoch in range(args.epochs):
        sampler.reset()
        for batch in sampler:
            x = torch.as_tensor(batch["x"], dtype=torch.float32).to(dev)
            y = torch.as_tensor(batch["y"]).to(dev)
            if dev.type == "cuda":
                x = x.to(torch.bfloat16)
            opt.zero_grad()
            loss = softmax_cross_entropy(model(x).float(), y)
            loss.backward()
            opt.step()
            clips += len(y)
            steps += 1
            if args.max_steps and steps >= args.max_steps:
                break
        if args.max_steps and steps >= args.max_steps:
            break
    if dev.type == "cuda":
        torch.cuda.synchronize()
    if group.rank == 0:
        print("%s: %d clips in %d steps, %.2f clips/s per rank, last loss %.4f, frames per clip %d..%d"
              % (args.mode, clips, steps, clips / (time.time() - t0), float(loss.detach()), train.lengths.min(),
                 train.lengths.max()))
    opt.close()
    es.finalize()


if __name__ == "__main__":
    main()
