"""The allocation-free batch-norm entry point, called through its exported C symbol.

Some users of the kernel library cannot allocate device memory when they need the op — the
GPU is owned by another allocator, or an allocation's device-wide synchronisation is not
acceptable, or they are plain C programs without a tensor library.  For them
``esgd_bn_forward_noalloc`` keeps its per-channel work arrays in a fixed block inside the
library.  This test loads the shared library directly, calls the symbol twice in a row on
different data (the block is shared between calls and must be re-initialised by the callee)
and compares each result with the regular three-call path whose work arrays the caller
allocates, and with PyTorch's fp32 ``batch_norm`` on the same data.  It also checks that an
oversized layer, a channel count that is not a multiple of 8 and a pointer that is not on a
16-byte boundary are refused with a readable message.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _load():
    from eagersgd_b200 import _build
    lib = C.CDLL(_build.build_cuda())
    vp = C.c_void_p
    lib.esgd_bn_forward_noalloc.restype = C.c_int
    lib.esgd_bn_forward_noalloc.argtypes = [vp, vp, vp, vp, vp, vp, vp, C.c_int64, C.c_int, C.c_int, C.c_float,
                                            C.c_float, vp]
    lib.esgd_bn_forward_noalloc_strerror.restype = C.c_char_p
    lib.esgd_bn_forward_noalloc_strerror.argtypes = [C.c_int]
    return lib


def _regular(y, res, gamma, beta, rm, rv, relu, momentum):
    """The existing entry points, with caller-allocated work arrays (through the ops layer)."""
    from eagersgd_b200.ops import functional as ops
    with torch.no_grad():
        return ops.bn_act(y, gamma, beta, rm, rv, momentum, relu, res)


@pytest.mark.parametrize("with_residual", [False, True])
def test_noalloc_matches_regular_path_twice_in_a_row(with_residual):
    lib = _load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    torch.manual_seed(0)
    stream = torch.cuda.current_stream(dev).cuda_stream
    # later calls: other shapes, same block; 264 channels = 33 groups of 8, which do not divide a block of 256 threads
    for call, (n, c, h, w) in enumerate([(8, 256, 14, 14), (4, 64, 9, 7), (3, 264, 5, 6)]):
        y = (torch.randn(n, c, h, w, device=dev) * 1.5 + 0.3).to(torch.bfloat16).contiguous(
            memory_format=torch.channels_last)
        res = torch.randn_like(y) if with_residual else None
        gamma = torch.rand(c, device=dev) + 0.5
        beta = torch.randn(c, device=dev)
        rm_a, rv_a = torch.zeros(c, device=dev), torch.ones(c, device=dev)
        rm_b, rv_b = torch.zeros(c, device=dev), torch.ones(c, device=dev)
        expect = _regular(y, res, gamma, beta, rm_a, rv_a, True, 0.1)
        y2d = y.permute(0, 2, 3, 1).reshape(-1, c)
        r2d = res.permute(0, 2, 3, 1).reshape(-1, c) if with_residual else None
        z2d = torch.empty_like(y2d)
        rc = lib.esgd_bn_forward_noalloc(y2d.data_ptr(), r2d.data_ptr() if with_residual else None, z2d.data_ptr(),
                                         gamma.data_ptr(), beta.data_ptr(), rm_b.data_ptr(), rv_b.data_ptr(),
                                         y2d.shape[0], c, 1, 0.1, 1e-5, stream)
        assert rc == 0, lib.esgd_bn_forward_noalloc_strerror(rc).decode()
        torch.cuda.synchronize()
        got = z2d.view(n, h, w, c).permute(0, 3, 1, 2)
        assert torch.allclose(got.float(), expect.float(), rtol=2e-2, atol=3e-2), call
        # fp32 oracle: PyTorch's batch norm on the same bf16 inputs, then residual and ReLU
        rm_c, rv_c = torch.zeros(c, device=dev), torch.ones(c, device=dev)
        ref = torch.nn.functional.batch_norm(y.float(), rm_c, rv_c, gamma, beta, True, 0.1, 1e-5)
        if with_residual:
            ref = ref + res.float()
        ref = torch.relu(ref)
        assert torch.allclose(got.float(), ref, rtol=1e-2, atol=2e-2), call
        assert torch.allclose(rm_b, rm_c, rtol=1e-3, atol=1e-3) and torch.allclose(rv_b, rv_c, rtol=1e-3, atol=1e-3)
        assert torch.allclose(rm_b, rm_a, rtol=1e-3, atol=1e-3) and torch.allclose(rv_b, rv_a, rtol=1e-3, atol=1e-3)


def test_noalloc_rejects_sizes_beyond_its_block():
    lib = _load()
    dev = torch.device("cuda", 0)
    c = 4096 + 8
    y = torch.zeros(16, c, dtype=torch.bfloat16, device=dev)
    z = torch.empty_like(y)
    g = torch.ones(c, device=dev)
    rc = lib.esgd_bn_forward_noalloc(y.data_ptr(), None, z.data_ptr(), g.data_ptr(), g.data_ptr(), None, None, 16, c,
                                     0, 0.1, 1e-5, torch.cuda.current_stream(dev).cuda_stream)
    assert rc == -2
    assert b"4096" in lib.esgd_bn_forward_noalloc_strerror(rc)
    rc = lib.esgd_bn_forward_noalloc(y.data_ptr(), None, z.data_ptr(), g.data_ptr(), g.data_ptr(), None, None, 16, 12,
                                     0, 0.1, 1e-5, torch.cuda.current_stream(dev).cuda_stream)
    assert rc == -1
    # a pointer into the middle of a 16-byte vector is refused on the host instead of faulting on the device
    c = 64
    y = torch.zeros(16 * c + 8, dtype=torch.bfloat16, device=dev)
    z = torch.empty_like(y)
    g = torch.ones(c, device=dev)
    for yp, zp in ((y.data_ptr() + 2, z.data_ptr()), (y.data_ptr(), z.data_ptr() + 8)):
        rc = lib.esgd_bn_forward_noalloc(yp, None, zp, g.data_ptr(), g.data_ptr(), None, None, 16, c, 0, 0.1, 1e-5,
                                         torch.cuda.current_stream(dev).cuda_stream)
        assert rc == -1
    assert b"16-byte" in lib.esgd_bn_forward_noalloc_strerror(-1)
