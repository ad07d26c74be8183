"""Train an ImageNet-sized ResNet on synthetic input and report images per second: the input pipeline is out of
the picture, what remains is the model, the optimizer and (with several ranks) the collective.

    python samples/synthetic_dataset.py [--resnet-size 50] [--batch 64] [--steps 20] [--mode solo]
    torchrun --nproc-per-node 8 samples/synthetic_dataset.py --mode majority

Counterpart of deep500 samples/synthetic_dataset.py (fixed random batch, time per step, optional Horovod).
"""
import argparse
import time
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch  # noqa: E402

import eagersgd_b200 as es  # noqa: E402
from eagersgd_b200.data import SyntheticImageNet  # noqa: E402
from eagersgd_b200.models.resnet import cifar_resnet, imagenet_resnet  # noqa: E402
from eagersgd_b200.train.step import TrainStep  # noqa: E402


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--resnet-size", type=int, default=50)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--size", type=int, default=224)
    ap.add_argument("--mode", default="solo", choices=["solo", "majority", "sync"])
    args = ap.parse_args(argv)
    group = es.init()
    dev = group.device
    torch.manual_seed(0)
    small = args.resnet_size < 18
    model = cifar_resnet(args.resnet_size, 1, 10) if small else imagenet_resnet(args.resnet_size, 1, 1000)
    ds = SyntheticImageNet(size=args.size, classes=10 if small else 1000)
    b = ds[list(range(args.batch))]
    x = torch.as_tensor(b["x"].copy())
    y = torch.as_tensor(b["y"])
    step = TrainStep(model, group, mode=args.mode, lr=0.01)
    x = x.to(dev)
    if dev.type == "cuda":
        x = x.to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    y = y.to(dev)
    for _ in range(3):
        step.run_device(x, y)
    if dev.type == "cuda":
        torch.cuda.synchronize()
    group.barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        loss = step.run_device(x, y)
    if dev.type == "cuda":
        torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    if group.rank == 0:
        print("ResNet-%d, batch %d x %d ranks, %s: %.1f images/s, %.2f ms/step, loss %.3f"
              % (args.resnet_size, args.batch, group.world, args.mode, group.world * args.batch * args.steps / dt,
                 1e3 * dt / args.steps, float(loss)))
    step.close()
    es.finalize()
    return dt


if __name__ == "__main__":
    main()
