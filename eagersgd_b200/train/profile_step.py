"""Per-kernel time shares of one training step.

    python -m eagersgd_b200.train.profile_step --model resnet50 --batch 256 [--steps 3] [--rows 40]

Runs ``--steps`` eager (not graph-replayed) steps of the flagship ``TrainStep`` under ``torch.profiler`` after a
warm-up and prints device time per kernel and step, largest first.  It is the step-level counterpart of the
kernel micro-benchmarks (``ops/bench_ops.py``) and of the reference's benchmark logger / ``CommProfiling`` metric
(official/utils/logs/logger.py; deep500/lv3/metrics.py).  Kernel times are what the profiler attributes to each
launch; use them as shares of the step, and ``bench.py`` for the step time itself.
"""
from __future__ import annotations

import argparse
import re
import sys

import torch


def kernel_table(prof, steps: int, rows: int):
    out = []
    for e in prof.key_averages():
        t = getattr(e, "self_device_time_total", None)
        if t is None:
            t = getattr(e, "self_cuda_time_total", 0.0)
        name = e.key
        if t <= 0 or name.startswith("autograd::") or name.startswith("aten::") or re.match(r"^_[A-Z]", name):
            continue                                   # keep kernels, drop operator / autograd wrappers
        out.append((t / 1e3 / steps, name, e.count // max(steps, 1)))
    out.sort(reverse=True)
    return out[:rows], sum(v for v, _, _ in out)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="resnet50", choices=["resnet50", "resnet32"])
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--rows", type=int, default=40)
    args = ap.parse_args(argv)
    assert torch.cuda.is_available(), "needs a CUDA device"
    import eagersgd_b200 as es
    from eagersgd_b200.models.resnet import cifar_resnet, imagenet_resnet
    from eagersgd_b200.train.step import TrainStep
    from torch.profiler import ProfilerActivity, profile
    group = es.Group()
    torch.manual_seed(0)
    if args.model == "resnet50":
        model, shape, classes = imagenet_resnet(50, 1, 1000), (args.batch, 3, 224, 224), 1000
    else:
        model, shape, classes = cifar_resnet(32), (args.batch, 3, 32, 32), 10
    step = TrainStep(model, group, mode="solo")
    x = torch.randn(*shape, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    y = torch.randint(0, classes, (args.batch,), device="cuda")
    for _ in range(3):
        step.run_device(x, y)
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        for _ in range(args.steps):
            step.run_device(x, y)
        torch.cuda.synchronize()
    table, total = kernel_table(prof, args.steps, args.rows)
    print("device time per step, by kernel (sum %.2f ms over all kernels)" % total)
    for ms, name, calls in table:
        print("%8.3f ms  %5.1f %%  %4d launches  %s" % (ms, 100.0 * ms / total, calls, name[:110]))
    return 0


if __name__ == "__main__":
    sys.exit(main())
