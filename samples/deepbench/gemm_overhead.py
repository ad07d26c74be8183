"""DeepBench GEMM sizes: the framework-level operator (autograd function, checks, launch) against the bare
kernel call and against PyTorch's matmul — how much the layers above the kernel cost.

    python samples/deepbench/gemm_overhead.py [--reruns 20] [--limit 5]

Counterpart of deep500 samples/deepbench/gemm_overhead_pytorch.py:30-125 (native op vs Deep500 wrapper).
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
    args = ap.parse_args(argv)
    dev = torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
    dt = torch.bfloat16 if dev.type == "cuda" else torch.float32
    from eagersgd_b200.ops import functional as ops
    rows = []
    for (m, n, k, ta, tb) in problems.GEMM[:args.limit or None]:
        a = torch.randn((k, m) if ta else (m, k), device=dev, dtype=dt)
        b = torch.randn((n, k) if tb else (k, n), device=dev, dtype=dt)
        A = a.t() if ta else a
        B = b.t() if tb else b
        w = B.t().contiguous()                                    # [N, K]: the layout of a dense layer's weight
        t_torch = timed(lambda: A @ B, args.reruns, dev)
        t_ours = timed(lambda: ops.linear(A.contiguous(), w, None), args.reruns, dev)
        flops = 2.0 * m * n * k
        rows.append((m, n, k, ta, tb, t_torch, t_ours))
        print("M %5d N %5d K %5d %s%s  torch %.3f ms (%.1f TFLOP/s)  ours %.3f ms (%.1f TFLOP/s)  ratio %.2f"
              % (m, n, k, "T" if ta else "N", "T" if tb else "N", 1e3 * t_torch, flops / t_torch / 1e12,
                 1e3 * t_ours, flops / t_ours / 1e12, t_ours / t_torch))
    return rows


if __name__ == "__main__":
    main()
