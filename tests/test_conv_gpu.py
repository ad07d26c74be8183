"""Implicit-GEMM convolution (tcgen05 + 4-D TMA) against PyTorch fp32 convolution."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _cl(x):
    return x.contiguous(memory_format=torch.channels_last)


CASES = [  # n, cin, h, w, cout, k, stride, pad
    (2, 64, 56, 56, 64, 3, 1, 1),
    (3, 128, 28, 28, 128, 3, 1, 1),
    (4, 256, 14, 14, 256, 3, 1, 1),
    (5, 512, 7, 7, 512, 3, 1, 1),
    (2, 64, 16, 24, 72, 3, 1, 1),
    (2, 128, 56, 56, 128, 3, 2, 1),
    (3, 256, 28, 28, 256, 3, 2, 1),
    (2, 512, 14, 14, 512, 3, 2, 1),
    (1, 64, 130, 130, 64, 3, 1, 1),
    (2, 64, 20, 20, 64, 5, 1, 2),
    (16, 64, 56, 56, 64, 3, 1, 1),     # enough tiles per CTA for the filter bank to stay in shared memory
    (20, 64, 112, 112, 64, 3, 2, 1),   # the same with stride 2
]


@pytest.mark.parametrize("n,cin,h,w,cout,k,stride,pad", CASES)
def test_conv_forward(n, cin, h, w, cout, k, stride, pad):
    from eagersgd_b200.ops import functional as ops
    from eagersgd_b200.ops.gemm import check_error
    torch.manual_seed(n * 7 + cin + h)
    x = _cl(torch.randn(n, cin, h, w, device=DEV)).to(torch.bfloat16)
    wt = _cl(torch.randn(cout, cin, k, k, device=DEV) * (1.0 / (k * cin ** 0.5))).to(torch.bfloat16)
    y, stats = ops.conv2d(x, wt, stride, pad, want_stats=True)
    torch.cuda.synchronize()
    check_error(x.device)
    ref = F.conv2d(x.float(), wt.float(), None, stride, pad)
    assert y.shape == ref.shape
    err = (y.float() - ref).abs().max().item()
    assert err < 3e-2 * max(1.0, ref.abs().max().item()), err
    assert stats is not None
    yf = y.float()
    assert torch.allclose(stats[0], yf.sum((0, 2, 3)), rtol=1e-3, atol=0.5)
    assert torch.allclose(stats[1], (yf * yf).sum((0, 2, 3)), rtol=1e-3, atol=0.5)


@pytest.mark.parametrize("n,cin,h,w,cout,k,stride,pad", [CASES[0], CASES[2], CASES[3], CASES[5]])
def test_conv_backward(n, cin, h, w, cout, k, stride, pad):
    from eagersgd_b200.ops import functional as ops
    torch.manual_seed(11)
    x = _cl(torch.randn(n, cin, h, w, device=DEV)).to(torch.bfloat16).requires_grad_()
    wt = _cl(torch.randn(cout, cin, k, k, device=DEV) * (1.0 / (k * cin ** 0.5))).to(torch.bfloat16).requires_grad_()
    y, _ = ops.conv2d(x, wt, stride, pad)
    g = _cl(torch.randn_like(y.float())).to(torch.bfloat16)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(), wt.detach().float().requires_grad_()
    F.conv2d(xr, wr, None, stride, pad).backward(g.float())
    assert torch.allclose(x.grad.float(), xr.grad, rtol=3e-2, atol=3e-2 * xr.grad.abs().max().item())
    assert torch.allclose(wt.grad.float(), wr.grad, rtol=3e-2, atol=3e-2 * wr.grad.abs().max().item())


@pytest.mark.parametrize("n,cin,h,w,cout", [(2, 128, 28, 28, 128), (3, 64, 16, 24, 256)])
def test_conv_stride2_data_gradient_by_parity(n, cin, h, w, cout):
    from eagersgd_b200.ops import functional as ops
    from eagersgd_b200.ops.gemm import check_error
    torch.manual_seed(3)
    x = _cl(torch.randn(n, cin, h, w, device=DEV)).to(torch.bfloat16).requires_grad_()
    wt = _cl(torch.randn(cout, cin, 3, 3, device=DEV) * 0.05).to(torch.bfloat16).requires_grad_()
    y, _ = ops.conv2d(x, wt, 2, 1)
    g = _cl(torch.randn_like(y.float())).to(torch.bfloat16)
    y.backward(g)
    torch.cuda.synchronize()
    check_error(x.device)
    xr, wr = x.detach().float().requires_grad_(), wt.detach().float().requires_grad_()
    F.conv2d(xr, wr, None, 2, 1).backward(g.float())
    assert torch.allclose(x.grad.float(), xr.grad, rtol=3e-2, atol=3e-2 * xr.grad.abs().max().item())
    assert torch.allclose(wt.grad.float(), wr.grad, rtol=3e-2, atol=3e-2 * wr.grad.abs().max().item())


def test_stem_convolution_im2col_gemm():
    from eagersgd_b200.ops import functional as ops
    torch.manual_seed(4)
    x = _cl(torch.randn(4, 3, 64, 64, device=DEV)).to(torch.bfloat16)
    wt = _cl(torch.randn(64, 3, 7, 7, device=DEV) * 0.1).to(torch.bfloat16).requires_grad_()
    y, stats = ops.conv2d(x, wt, 2, 3, want_stats=True)
    g = _cl(torch.randn_like(y.float())).to(torch.bfloat16)
    y.backward(g)
    wr = wt.detach().float().requires_grad_()
    yr = F.conv2d(x.float(), wr, None, 2, 3)
    yr.backward(g.float())
    assert torch.allclose(y.float(), yr, rtol=3e-2, atol=5e-2)
    assert torch.allclose(stats[0], y.float().sum((0, 2, 3)), rtol=1e-3, atol=0.5)
    assert torch.allclose(wt.grad.float(), wr.grad, rtol=3e-2, atol=3e-2 * wr.grad.abs().max().item())


@pytest.mark.parametrize("n,cin,h,w,cout,k", [(8, 64, 56, 56, 64, 3), (6, 128, 28, 28, 128, 3), (4, 128, 14, 14, 64, 3),
                                              (3, 64, 24, 24, 128, 5)])
def test_halo_views_match_per_tap_loads(n, cin, h, w, cout, k, monkeypatch):
    """Stride-1 convolutions read one input box per channel block and take the taps as shifted views of it;
    the per-tap path (one TMA box per tap) is the same arithmetic in another order of the K steps."""
    from eagersgd_b200.ops import functional as ops
    from eagersgd_b200.ops.gemm import check_error
    torch.manual_seed(n + h)
    x = _cl(torch.randn(n, cin, h, w, device=DEV)).to(torch.bfloat16)
    wt = _cl(torch.randn(cout, cin, k, k, device=DEV) * (1.0 / (k * cin ** 0.5))).to(torch.bfloat16)
    pad = (k - 1) // 2
    y_halo, st_halo = ops.conv2d(x, wt, 1, pad, want_stats=True)
    monkeypatch.setenv("ESGD_CONV_HALO", "0")
    y_tap, st_tap = ops.conv2d(x, wt, 1, pad, want_stats=True)
    monkeypatch.delenv("ESGD_CONV_HALO")
    torch.cuda.synchronize()
    check_error(x.device)
    ref = F.conv2d(x.float(), wt.float(), None, 1, pad)
    assert (y_halo.float() - ref).abs().max().item() < 3e-2 * max(1.0, ref.abs().max().item())
    assert (y_halo.float() - y_tap.float()).abs().max().item() <= 2e-2 * max(1.0, ref.abs().max().item())
    assert torch.allclose(st_halo[0], y_halo.float().sum((0, 2, 3)), rtol=1e-3, atol=0.5)
    assert torch.allclose(st_halo, st_tap, rtol=2e-2, atol=2.0)


@pytest.mark.parametrize("n,cin,h,w,cout,k", [(8, 64, 56, 56, 64, 3), (6, 128, 28, 28, 128, 3), (5, 64, 28, 28, 256, 3),
                                              (3, 64, 24, 24, 72, 5), (40, 64, 56, 56, 64, 3), (12, 256, 14, 14, 256, 3),
                                              (16, 512, 7, 7, 512, 3)])
def test_weight_gradient_with_shared_boxes(n, cin, h, w, cout, k, monkeypatch):
    """Weight gradient from one dy box and one x box per block of rows (taps = shifted views) against the fp32
    reference and against the per-tap kernel."""
    from eagersgd_b200.ops import functional as ops
    from eagersgd_b200.ops.gemm import check_error
    torch.manual_seed(h + cout)
    x = _cl(torch.randn(n, cin, h, w, device=DEV)).to(torch.bfloat16)
    wt = _cl(torch.randn(cout, cin, k, k, device=DEV) * 0.05).to(torch.bfloat16).requires_grad_()
    pad = (k - 1) // 2
    y, _ = ops.conv2d(x, wt, 1, pad)
    g = _cl(torch.randn_like(y.float()) * 0.1).to(torch.bfloat16)
    (dw_shared,) = torch.autograd.grad(y, wt, g, retain_graph=True)
    monkeypatch.setenv("ESGD_CONV_HALO", "0")
    (dw_tap,) = torch.autograd.grad(y, wt, g, retain_graph=True)
    monkeypatch.delenv("ESGD_CONV_HALO")
    torch.cuda.synchronize()
    check_error(x.device)
    wr = wt.detach().float().requires_grad_()
    F.conv2d(x.float(), wr, None, 1, pad).backward(g.float())
    scale = wr.grad.abs().max().item()
    assert (dw_shared.float() - wr.grad).abs().max().item() < 2e-2 * scale
    assert (dw_shared.float() - dw_tap.float()).abs().max().item() < 2e-2 * scale


# ---- small shapes, every geometry the kernels accept, against the compiled C++ oracle ----------------------------
def _small_cases():
    cases = []
    for n in (1, 2):
        for (h, w) in ((5, 5), (8, 9), (9, 6)):
            for (cin, cout) in ((64, 64), (128, 64), (64, 72)):
                for (k, stride, pad) in ((3, 1, 1), (3, 1, 0), (3, 2, 1), (3, 2, 0), (5, 2, 2), (1, 1, 0), (1, 2, 0), (5, 1, 2), (3, 1, 2)):
                    if (h + 2 * pad - k) // stride + 1 < 1 or (w + 2 * pad - k) // stride + 1 < 1:
                        continue
                    cases.append((n, cin, h, w, cout, k, stride, pad))
    # the narrow layers of the CIFAR ResNets (channel-padded around the kernel)
    for (cin, cout, stride) in ((16, 16, 1), (16, 32, 2), (32, 32, 1), (32, 64, 2)):
        cases.append((2, cin, 8, 8, cout, 3, stride, 1))
        cases.append((1, cin, 7, 9, cout, 3, stride, 1))
    return cases


@pytest.mark.parametrize("n,cin,h,w,cout,k,stride,pad", _small_cases())
def test_small_shapes_forward_dgrad_wgrad_against_cpp_oracle(n, cin, h, w, cout, k, stride, pad):
    """Forward, data gradient and weight gradient of small, odd-sized problems, element by element against the
    plain-loop C++ convolution (ref/cpp/ops.cpp) on the same bf16-rounded operands: every element within 1 % of
    the tensor's largest magnitude.  A dropped filter tap at an image border, a wrong halo or a mis-strided
    gradient shows up here as an error of the size of the values themselves."""
    from eagersgd_b200.ops import functional as ops
    from eagersgd_b200.ops.gemm import check_error
    from eagersgd_b200.ref import cpp_ops as R
    torch.manual_seed(n * 1000 + cin + 7 * h + w + k + stride)
    x = _cl(torch.randn(n, cin, h, w, device=DEV)).to(torch.bfloat16).requires_grad_()
    wt = _cl(torch.randn(cout, cin, k, k, device=DEV) * (1.0 / (k * cin ** 0.5))).to(torch.bfloat16).requires_grad_()
    y, _ = ops.conv2d(x, wt, stride, pad)
    g = _cl(torch.randn_like(y.float())).to(torch.bfloat16)
    y.backward(g)
    torch.cuda.synchronize()
    check_error(x.device)
    xn, wn, gn = x.detach().float().cpu().numpy(), wt.detach().float().cpu().numpy(), g.float().cpu().numpy()
    y_ref = R.conv2d(xn, wn, stride, pad)
    dx_ref, dw_ref = R.conv2d_grads(xn, wn, gn, stride, pad)
    for name, got, ref in (("y", y, y_ref), ("dx", x.grad, dx_ref), ("dw", wt.grad, dw_ref)):
        got = got.detach().float().cpu().numpy()
        assert got.shape == ref.shape, name
        tol = 1e-2 * max(float(abs(ref).max()), 1e-6)
        worst = float(abs(got - ref).max())
        assert worst <= tol, (name, worst, tol)
