"""Micro-benchmarks of the hand-written kernels, one JSON line per case.

    python -m eagersgd_b200.ops.bench_ops --op gemm --shape 8192,8192,8192
    python -m eagersgd_b200.ops.bench_ops --op conv --shape 64,128,56,56,128,3,1      (N,Cin,H,W,Cout,k,stride)
    python -m eagersgd_b200.ops.bench_ops --op conv_wgrad --shape 64,128,28,28,128,3,1
    python -m eagersgd_b200.ops.bench_ops --op bn --shape 256,256,56,56 [--backward]
    python -m eagersgd_b200.ops.bench_ops --op lstm --shape 64,16,2048,2048              (T,B,I,H)
    python -m eagersgd_b200.ops.bench_ops --op suite

Timing: 3 warm-up calls, then ``--iters`` calls between CUDA events on the launching stream with a
synchronise on both sides; between timed calls a buffer larger than L2 is overwritten so every call
starts cold.  Each line reports achieved TFLOP/s or GB/s and the fraction of the measured peak of
this machine (``MEASURED_PEAKS.json`` beside the repository root when present, else the stated
fallback), next to the same op through PyTorch's library path for comparison.  It stands where the
reference has its DeepBench-style loops (deep500 samples/deepbench/*.py).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.nn.functional as F

_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks():
    path = os.path.join(_ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


_flush = None


def flush_l2():
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")   # 256 MiB > 126 MB L2
    _flush.zero_()


def timeit(fn, iters: int, flush: bool = True, graph: bool = True) -> float:
    """Mean device time of ``fn`` in ms.  The call is captured in a CUDA graph first so that the
    measurement is the kernels' time, not the Python launch path (that is how a training step runs
    them, too)."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    if graph:
        try:
            g = torch.cuda.CUDAGraph()
            cur = torch.cuda.current_stream()
            # Capture on the stream the tensors were created on (main() runs everything on one side stream): a
            # gradient taken with respect to a leaf created on another stream makes autograd synchronise the two
            # streams, which is not allowed inside a capture.
            with (torch.cuda.graph(g, stream=cur) if cur != torch.cuda.default_stream() else torch.cuda.graph(g)):
                fn()
            fn = g.replay
            fn()
            torch.cuda.synchronize()
        except Exception as exc:   # time the plain launches instead, and say so
            print("graph capture failed, timing eager launches: %s" % str(exc).splitlines()[0], file=sys.stderr)
            torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush:
            flush_l2()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters


def _cl(x):
    return x.contiguous(memory_format=torch.channels_last)


def bench_gemm(shape, iters, a_k=True, b_k=True):
    from .gemm import gemm, check_error
    M, N, K = shape
    a = torch.randn((M, K) if a_k else (K, M), device="cuda").to(torch.bfloat16)
    b = torch.randn((N, K) if b_k else (K, N), device="cuda").to(torch.bfloat16)
    c = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    ms = timeit(lambda: gemm(a, b, a_kmajor=a_k, b_kmajor=b_k, out=c), iters)
    A = a if a_k else a.t()
    Bt = b.t() if b_k else b
    ms_lib = timeit(lambda: torch.matmul(A, Bt, out=c), iters)
    check_error(a.device)
    flops, byts = 2.0 * M * N * K, 2.0 * (M * K + N * K + M * N)
    return dict(op="gemm", M=M, N=N, K=K, ms=ms, tflops=flops / ms / 1e9, gbs=byts / ms / 1e6, library_ms=ms_lib)


def bench_conv(shape, iters, backward=False):
    from . import functional as ops
    n, cin, h, w, cout, k, stride = shape
    x = _cl(torch.randn(n, cin, h, w, device="cuda")).to(torch.bfloat16).requires_grad_(backward)
    wt = _cl(torch.randn(cout, cin, k, k, device="cuda") * 0.05).to(torch.bfloat16)
    pad = (k - 1) // 2
    y, _ = ops.conv2d(x, wt, stride, pad, want_stats=not backward)
    ho, wo = y.shape[2], y.shape[3]
    flops = 2.0 * n * ho * wo * cout * cin * k * k
    byts = 2.0 * (x.numel() + wt.numel() + y.numel())
    if backward:
        g = _cl(torch.randn_like(y.float())).to(torch.bfloat16)
        fn = lambda: torch.autograd.grad(ops.conv2d(x, wt, stride, pad)[0], x, g)
        with ops.reference_ops():
            lib = lambda: torch.autograd.grad(ops.conv2d(x, wt, stride, pad)[0], x, g)
            ms_lib = timeit(lib, iters, graph=False)
        ms = timeit(fn, iters)
        flops *= 2
    else:
        ms = timeit(lambda: ops.conv2d(x, wt, stride, pad, want_stats=True), iters)
        ms_lib = timeit(lambda: F.conv2d(x, wt, None, stride, pad), iters)
    return dict(op="conv_fwd+dgrad" if backward else "conv_fwd+stats", N=n, Cin=cin, H=h, W=w, Cout=cout, k=k,
                stride=stride, ms=ms, tflops=flops / ms / 1e9, gbs=byts / ms / 1e6, library_ms=ms_lib)


def bench_conv_wgrad(shape, iters):
    """Weight gradient of a k x k convolution (pixels are the reduction dimension)."""
    from . import functional as ops
    n, cin, h, w, cout, k, stride = shape
    x = _cl(torch.randn(n, cin, h, w, device="cuda")).to(torch.bfloat16)
    wt = _cl(torch.randn(cout, cin, k, k, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_()
    pad = (k - 1) // 2
    y, _ = ops.conv2d(x, wt, stride, pad)
    g = _cl(torch.randn_like(y.float())).to(torch.bfloat16)
    ms = timeit(lambda: torch.autograd.grad(y, wt, g, retain_graph=True), iters)
    with ops.reference_ops():
        y2, _ = ops.conv2d(x, wt, stride, pad)
        ms_lib = timeit(lambda: torch.autograd.grad(y2, wt, g, retain_graph=True), iters, graph=False)
    flops = 2.0 * n * y.shape[2] * y.shape[3] * cout * cin * k * k
    byts = 2.0 * (x.numel() + y.numel()) + 4.0 * wt.numel()
    return dict(op="conv_wgrad", N=n, Cin=cin, H=h, W=w, Cout=cout, k=k, stride=stride, ms=ms,
                tflops=flops / ms / 1e9, gbs=byts / ms / 1e6, library_ms=ms_lib)


def bench_bn(shape, iters, backward=False, residual=False):
    from . import functional as ops
    n, c, h, w = shape
    y = _cl(torch.randn(n, c, h, w, device="cuda")).to(torch.bfloat16).requires_grad_()
    res = torch.randn_like(y) if residual else None
    gamma = torch.ones(c, device="cuda", requires_grad=True)
    beta = torch.zeros(c, device="cuda", requires_grad=True)
    rm, rv = torch.zeros(c, device="cuda"), torch.ones(c, device="cuda")
    nb = y.numel() * 2.0
    if backward:
        z = ops.bn_act(y, gamma, beta, rm, rv, 0.1, True, res)
        dz = torch.randn_like(z)
        ms = timeit(lambda: torch.autograd.grad(z, (y, gamma, beta), dz, retain_graph=True), iters)
        byts = nb * ((2 + (1 if residual else 0)) + (3 + (2 if residual else 0)))   # reduce reads + apply reads/writes
        with ops.reference_ops():
            z2 = ops.bn_act(y, gamma, beta, rm, rv, 0.1, True, res)
            ms_lib = timeit(lambda: torch.autograd.grad(z2, (y, gamma, beta), dz, retain_graph=True), iters,
                            graph=False)
    else:
        ms = timeit(lambda: ops.bn_act(y, gamma, beta, rm, rv, 0.1, True, res), iters)
        byts = nb * (3 + (1 if residual else 0))      # stats read, apply read (+residual), write
        with ops.reference_ops(), torch.no_grad():
            ms_lib = timeit(lambda: ops.bn_act(y, gamma, beta, rm, rv, 0.1, True, res), iters)
    return dict(op="bn_relu_bwd" if backward else "bn_relu_fwd", N=n, C=c, H=h, W=w, residual=residual, ms=ms,
                gbs=byts / ms / 1e6, library_ms=ms_lib)


def bench_ce(shape, iters):
    from . import functional as ops
    b, c = shape
    logits = torch.randn(b, c, device="cuda").requires_grad_()
    labels = torch.randint(0, c, (b,), device="cuda")
    ms = timeit(lambda: ops.softmax_cross_entropy(logits, labels), iters, flush=False)
    ms_lib = timeit(lambda: F.cross_entropy(logits, labels), iters, flush=False)
    return dict(op="softmax_ce_fwd+grad", B=b, C=c, ms=ms, gbs=3 * b * c * 4.0 / ms / 1e6, library_ms=ms_lib)


def bench_lstm(shape, iters):
    """One LSTM layer, forward + backward: T steps of batch B, input I, hidden H (recurrent GEMM with swapped
    operands + fused gate kernel per step) against torch.nn.LSTM (cuDNN)."""
    from .lstm import lstm_layer
    T, B, I, H = shape
    x = torch.randn(T, B, I, device="cuda").to(torch.bfloat16).requires_grad_()
    w_ih = (torch.randn(4 * H, I, device="cuda") * 0.02).to(torch.bfloat16).requires_grad_()
    w_hh = (torch.randn(4 * H, H, device="cuda") * 0.02).to(torch.bfloat16).requires_grad_()
    bias = torch.zeros(4 * H, device="cuda", requires_grad=True)
    g = torch.randn(T, B, H, device="cuda").to(torch.bfloat16)
    ms = timeit(lambda: torch.autograd.grad(lstm_layer(x, w_ih, w_hh, bias), (x, w_ih, w_hh), g), iters, graph=False)
    ref = torch.nn.LSTM(I, H).cuda().to(torch.bfloat16)
    ms_lib = timeit(lambda: torch.autograd.grad(ref(x)[0], (x,) + tuple(ref.parameters()), g), iters, graph=False)
    flops = 3 * 2.0 * T * B * 4 * H * (I + H)
    byts = 3 * 2.0 * T * 4 * H * H                      # the recurrent weights are re-read every step, fwd and bwd
    return dict(op="lstm_layer_fwd+bwd", T=T, B=B, I=I, H=H, ms=ms, tflops=flops / ms / 1e9, gbs=byts / ms / 1e6,
                library_ms=ms_lib)


def bench_update(shape, iters):
    """The fused reduce + momentum-SGD kernel path of a single-rank channel (pack, control, update)."""
    from ..parallel.nvlink_channel import NvlinkChannel, create_arenas
    (count,) = shape
    dev = torch.device("cuda", torch.cuda.current_device())
    arena, bases = create_arenas(count, torch.bfloat16, 0, 1)
    grad = torch.randn(count, device=dev).to(torch.bfloat16)
    w32, mom = torch.randn(count, device=dev), torch.zeros(count, device=dev)
    w16 = w32.to(torch.bfloat16)
    hyper = torch.tensor([0.1, 0.9, 1e-4, 0, 1, 0, 0, 0], dtype=torch.float32, device=dev)
    ch = NvlinkChannel(count, 0, 1, bases, dev, grad, slot_dtype=torch.bfloat16, mode="solo", limiter=32, w32=w32,
                       mom=mom, w16=w16, hyper=hyper)
    ms = timeit(lambda: ch.step(), iters, graph=False)
    byts = count * (2 + 2 + 2 + 4 + 4 + 4 + 4 + 2.0)   # grad read, slot write+read, w32/mom read+write, w16 write
    torch.cuda.synchronize()
    arena.free()
    return dict(op="publish+reduce+fused_sgd(world=1)", count=count, ms=ms, gbs=byts / ms / 1e6)


def bench_lars(shape, iters):
    """Fused LARS (per-tensor norms kernel + trust-ratio update kernel) over the parameter tensors of ResNet-50,
    bf16 parameters with fp32 masters, against the per-tensor PyTorch LARS on fp32 copies."""
    from ..models.resnet import imagenet_resnet
    from ..optim.lars import LARS, FusedLARS
    (depth,) = shape
    dev = torch.device("cuda", torch.cuda.current_device())
    model = imagenet_resnet(depth).to(dev)
    ref = [torch.nn.Parameter(p.detach().clone()) for p in model.parameters()]
    for p in model.parameters():
        p.data = p.data.to(torch.bfloat16)
    params = list(model.parameters())
    fused = FusedLARS(params, lr=0.1, momentum=0.9, weight_decay=1e-4, eeta=0.001)
    plain = LARS(ref, lr=0.1, momentum=0.9, weight_decay=1e-4, eeta=0.001)
    for p, q in zip(params, ref):
        p.grad.normal_() if p.grad is not None else None
        q.grad = torch.randn_like(q)
    count = sum(p.numel() for p in params)
    ms = timeit(lambda: fused.step(), iters, graph=False)
    ms_lib = timeit(lambda: plain.step(), iters, graph=False)
    byts = count * (2 + 4 + 2 + 4 + 4 + 4 + 4 + 2.0)    # norms: grad + w32; update: grad, w32 / momentum read + write, bf16 copy
    return dict(op="fused_lars", tensors=len(params), count=count, ms=ms, gbs=byts / ms / 1e6, library_ms=ms_lib)


SUITE = [("gemm", (8192, 8192, 8192)), ("gemm", (4096, 4096, 4096)), ("gemm", (802816, 64, 256)),
         ("gemm", (802816, 256, 64)), ("gemm", (200704, 512, 128)), ("gemm", (50176, 1024, 256)),
         ("gemm", (12544, 2048, 512)), ("conv", (256, 64, 56, 56, 64, 3, 1)), ("conv", (256, 128, 28, 28, 128, 3, 1)),
         ("conv", (256, 256, 14, 14, 256, 3, 1)), ("conv", (256, 512, 7, 7, 512, 3, 1)),
         ("conv", (256, 128, 56, 56, 128, 3, 2)), ("bn", (256, 64, 112, 112)), ("bn", (256, 256, 56, 56)),
         ("bn", (256, 1024, 14, 14)), ("ce", (256, 1000)), ("update", (25557032 // 8 * 8,))]


def run(op, shape, iters, backward=False, residual=False):
    if op == "gemm":
        r = bench_gemm(shape, iters)
    elif op == "gemm_wgrad":
        r = bench_gemm(shape, iters, False, False)
    elif op == "conv":
        r = bench_conv(shape, iters, backward)
    elif op == "conv_wgrad":
        r = bench_conv_wgrad(shape, iters)
    elif op == "bn":
        r = bench_bn(shape, iters, backward, residual)
    elif op == "ce":
        r = bench_ce(shape, iters)
    elif op == "lstm":
        r = bench_lstm(shape, iters)
    elif op == "update":
        r = bench_update(shape, iters)
    elif op == "lars":
        r = bench_lars(shape, iters)
    else:
        raise SystemExit("unknown op " + op)
    p = peaks()
    if "tflops" in r:
        r["frac_of_%s_bf16_peak" % p["source"]] = r["tflops"] / p["bf16_tflops"]
    r["frac_of_%s_hbm_peak" % p["source"]] = r["gbs"] / p["hbm_gbs"]
    return r


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="suite")
    ap.add_argument("--shape", default="")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--backward", action="store_true")
    ap.add_argument("--residual", action="store_true")
    args = ap.parse_args(argv)
    assert torch.cuda.is_available(), "the kernels need a CUDA device"
    with torch.cuda.stream(torch.cuda.Stream()):      # tensors, warm-up, capture and replay share this stream
        return _run_cases(args)


def _run_cases(args):
    if args.op == "suite":
        for op, shape in SUITE:
            print(json.dumps(run(op, shape, args.iters)), flush=True)
            if op in ("conv", "bn"):
                print(json.dumps(run(op, shape, args.iters, backward=True)), flush=True)
    else:
        shape = tuple(int(v) for v in args.shape.split(","))
        print(json.dumps(run(args.op, shape, args.iters, args.backward, args.residual)), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
