"""DeepBench convolution sizes, forward and backward: this framework's convolution operator against PyTorch's.

    python samples/deepbench/conv_overhead.py [--reruns 20] [--limit 5] [--backward]

Counterpart of deep500 samples/deepbench/conv_overhead_pytorch.py:25-95.
"""
import argparse
import time
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import torch  # noqa: E402

from samples.deepbench import problems  # noqa: E402


def timed(fn, reruns, dev):
    """Median seconds of ``reruns`` calls, synchronising around each on a GPU (host time alone would measure
    the launch, not the work)."""
    out = []
    for _ in range(reruns):
        if dev.type == "cuda":
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        fn()
        if dev.type == "cuda":
            torch.cuda.synchronize()
        out.append(time.perf_counter() - t0)
    out.sort()
    return out[len(out) // 2]


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--reruns", type=int, default=20)
    ap.add_argument("--limit", type=int, default=0)
    ap.add_argument("--backward", action="store_true")
    args = ap.parse_args(argv)
    dev = torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
    dt = torch.bfloat16 if dev.type == "cuda" else torch.float32
    from eagersgd_b200.ops import functional as ops
    rows = []
    for (w_, h_, c, n, k, s, r, pw, ph, sw, sh) in problems.CONV[:args.limit or None]:
        x = torch.randn(n, c, h_, w_, device=dev, dtype=dt).contiguous(memory_format=torch.channels_last).requires_grad_(args.backward)
        wt = torch.randn(k, c, r, s, device=dev, dtype=dt).contiguous(memory_format=torch.channels_last).requires_grad_(args.backward)

        def run(fn):
            y = fn()
            y = y[0] if isinstance(y, tuple) else y
            if args.backward:
                y.float().sum().backward()
        t_torch = timed(lambda: run(lambda: torch.nn.functional.conv2d(x, wt, stride=sh, padding=ph)), args.reruns, dev)
        t_ours = timed(lambda: run(lambda: ops.conv2d(x, wt, sh, ph)), args.reruns, dev)
        rows.append((w_, h_, c, n, k, r, t_torch, t_ours))
        print("%3dx%-3d C %4d N %2d K %4d %dx%d /%d  torch %.3f ms  ours %.3f ms  ratio %.2f"
              % (h_, w_, c, n, k, r, s, sh, 1e3 * t_torch, 1e3 * t_ours, t_ours / t_torch))
    return rows


if __name__ == "__main__":
    main()
