"""Sequence classification with variable-length clips: the eager-SGD LSTM workload.

    torchrun --nproc-per-node 8 samples/lstm_video_classifier.py --mode majority --steps 50

Per-frame 2048-d features (synthetic here), lengths from a clipped log-normal over 30..1800 frames,
length-bucketed batches of 16, a 2-layer LSTM (hidden 2048) and a 101-way head; the per-rank
sequence length is the natural load imbalance (deep500 samples/ucf101_resnetlstm.py:18-113).
"""
import argparse
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import eagersgd_b200 as es  # noqa: E402
from eagersgd_b200.data import BucketSampler, SyntheticSequenceDataset  # noqa: E402
from eagersgd_b200.models.lstm import LSTMClassifier  # noqa: E402
from eagersgd_b200.ops.functional import softmax_cross_entropy  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", default="majority", choices=["solo", "majority", "sync"])
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--max-length", type=int, default=500)
    ap.add_argument("--batch", type=int, default=16)
    args = ap.parse_args()
    group = es.init()
    dev = group.device
    torch.manual_seed(0)
    model = LSTMClassifier(2048, args.hidden, 2, 101).to(dev)
    if dev.type == "cuda":
        model.compute_dtype_(torch.bfloat16)
    ds = SyntheticSequenceDataset(4096, 2048, 101, seed=group.rank + 1)
    sampler = BucketSampler(ds, args.batch, ds.lengths, num_buckets=30, max_length=args.max_length, seed=group.rank)
    inner = torch.optim.SGD(model.parameters(), lr=0.05, momentum=0.9)
    cls = {"solo": es.SoloAllreduceOptimizer, "majority": es.MajorityAllreduceOptimizer, "sync": es.SyncAllreduceOptimizer}
    opt = cls[args.mode](inner, group)
    seqs, t0 = 0, time.time()
    for step in range(args.steps):
        batch = sampler()
        if batch is None:
            sampler.reset()
            batch = sampler()
        x = torch.as_tensor(batch["x"]).to(dev)
        y = torch.as_tensor(batch["y"]).to(dev)
        if dev.type == "cuda":
            x = x.to(torch.bfloat16)
        opt.zero_grad()
        loss = softmax_cross_entropy(model(x).float(), y)
        loss.backward()
        opt.step()
        seqs += len(y)
    if dev.type == "cuda":
        torch.cuda.synchronize()
    if group.rank == 0:
        print("mode %s: %.1f sequences/s per rank, last loss %.4f, stats %s"
              % (args.mode, seqs / (time.time() - t0), float(loss.detach()), opt.stats()))
    opt.close()
    es.finalize()


if __name__ == "__main__":
    main()
