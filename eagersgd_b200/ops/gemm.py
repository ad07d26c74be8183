"""bf16 GEMM on the 5th-generation tensor cores (tcgen05 + TMEM + TMA).

``gemm(a, b)`` computes ``a @ b.T``-style products with fp32 accumulation:

    C[M, N] = A[M, K] . B[N, K]^T

where either operand may instead be given in its transposed storage
(``a_kmajor=False`` means ``a`` is stored ``[K, M]``), which is the layout the
weight-gradient GEMMs over NHWC activations need.  There is no fallback path: on
a CUDA device the kernel library must load.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from ..parallel import _native as N

_err_flags = {}


def _lib():
    lib = N.cuda()
    if not getattr(lib, "_gemm_bound", False):
        lib.esgd_gemm_bf16.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p] + [C.c_int] * 9 + \
            [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
        lib._gemm_bound = True
    return lib


def error_flag(device: torch.device) -> torch.Tensor:
    """Per-device int32 word the tensor-core kernels raise when a bounded wait runs out."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _err_flags:
        _err_flags[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _err_flags[key]


def check_error(device: torch.device) -> None:
    if int(error_flag(device).item()) != 0:
        raise RuntimeError("a tensor-core kernel gave up on a bounded wait (pipeline stall)")


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_kmajor: bool = True, b_kmajor: bool = True,
         out: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16,
         bias: Optional[torch.Tensor] = None, relu: bool = False, splits: int = 1, accumulate: bool = False,
         col_sum: Optional[torch.Tensor] = None, col_sqsum: Optional[torch.Tensor] = None,
         residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``residual``: a bf16 ``[M, N]`` tensor added to the product in the epilogue, before the single
    rounding to bf16 (bf16 output only)."""
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.is_cuda
    assert a.dim() == 2 and b.dim() == 2 and a.stride(1) == 1 and b.stride(1) == 1
    if a_kmajor:
        M, K = a.shape
    else:
        K, M = a.shape
    if b_kmajor:
        Nn, Kb = b.shape
    else:
        Kb, Nn = b.shape
    assert K == Kb, "inner dimensions differ"
    atomic = splits > 1 or accumulate
    if out is None:
        dt = torch.float32 if atomic else out_dtype
        out = (torch.zeros if atomic else torch.empty)((M, Nn), dtype=dt, device=a.device)
    assert out.stride(1) == 1 and out.shape == (M, Nn)
    mode = 2 if atomic else (0 if out.dtype == torch.bfloat16 else 1)
    if atomic:
        assert out.dtype == torch.float32
    if residual is not None:
        assert residual.dtype == torch.bfloat16 and residual.shape == (M, Nn) and residual.stride(1) == 1 and mode == 0
    stream = torch.cuda.current_stream(a.device).cuda_stream
    rc = _lib().esgd_gemm_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, Nn, K, a.stride(0), b.stride(0),
                               out.stride(0), int(not a_kmajor), int(not b_kmajor), mode,
                               bias.data_ptr() if bias is not None else None, int(relu), splits,
                               col_sum.data_ptr() if col_sum is not None else None,
                               col_sqsum.data_ptr() if col_sqsum is not None else None,
                               residual.data_ptr() if residual is not None else None,
                               residual.stride(0) if residual is not None else 0,
                               error_flag(a.device).data_ptr(), stream)
    if rc != 0:
        raise RuntimeError("esgd_gemm_bf16 failed with code %d (M=%d N=%d K=%d)" % (rc, M, Nn, K))
    return out
