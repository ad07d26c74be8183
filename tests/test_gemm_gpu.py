"""tcgen05 GEMM against a plain PyTorch fp32 reference of the same product."""
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _ref(a, b, a_k, b_k):
    A = a.float() if a_k else a.float().t()
    B = b.float() if b_k else b.float().t()
    return A @ B.t()


def _rand(shape, scale=1.0):
    return (torch.randn(*shape, device=DEV) * scale).to(torch.bfloat16)


@pytest.mark.parametrize("M,N,K", [(128, 64, 64), (256, 128, 128), (512, 256, 512), (1000, 1000, 2048),
                                   (130, 72, 200), (3136, 64, 256), (4096, 512, 1024), (77, 2048, 64)])
def test_gemm_kmajor(M, N, K):
    from eagersgd_b200.ops.gemm import gemm, check_error
    torch.manual_seed(M + N + K)
    a, b = _rand((M, K)), _rand((N, K))
    c = gemm(a, b)
    torch.cuda.synchronize()
    check_error(a.device)
    ref = _ref(a, b, True, True)
    err = (c.float() - ref).abs().max().item()
    assert err <= 0.02 * ref.abs().max().item() + 1e-2, err


@pytest.mark.parametrize("a_k,b_k", [(True, False), (False, False), (False, True)])
@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (256, 64, 4096), (512, 256, 1000), (192, 320, 264)])
def test_gemm_transposed_storage(a_k, b_k, M, N, K):
    from eagersgd_b200.ops.gemm import gemm, check_error
    torch.manual_seed(1)
    a = _rand((M, K) if a_k else (K, M))
    b = _rand((N, K) if b_k else (K, N))
    c = gemm(a, b, a_kmajor=a_k, b_kmajor=b_k, out_dtype=torch.float32)
    torch.cuda.synchronize()
    check_error(a.device)
    ref = _ref(a, b, a_k, b_k)
    assert (c - ref).abs().max().item() <= 2e-3 * ref.abs().max().item() + 1e-3


def test_gemm_splitk_weight_gradient_shape():
    """dW[Cout,Cin] = dY^T . X over many pixels: both operands in [K][MN] storage, split-K atomics."""
    from eagersgd_b200.ops.gemm import gemm, check_error
    torch.manual_seed(2)
    pixels, cout, cin = 50000, 256, 64
    dy, x = _rand((pixels, cout), 0.1), _rand((pixels, cin), 0.1)
    dw = gemm(dy, x, a_kmajor=False, b_kmajor=False, splits=64)
    torch.cuda.synchronize()
    check_error(dy.device)
    ref = dy.float().t() @ x.float()
    assert (dw - ref).abs().max().item() <= 2e-3 * ref.abs().max().item() + 1e-3


def test_gemm_epilogue_bias_relu_stats():
    from eagersgd_b200.ops.gemm import gemm, check_error
    torch.manual_seed(3)
    M, N, K = 1024, 256, 320
    a, b = _rand((M, K)), _rand((N, K))
    bias = torch.randn(N, device=DEV)
    s = torch.zeros(N, device=DEV)
    s2 = torch.zeros(N, device=DEV)
    c = gemm(a, b, bias=bias, relu=True, out_dtype=torch.float32)
    cb = gemm(a, b, bias=bias, col_sum=s, col_sqsum=s2)      # bf16 output + statistics of the stored values
    torch.cuda.synchronize()
    check_error(a.device)
    pre = _ref(a, b, True, True) + bias
    assert torch.allclose(c, pre.relu(), rtol=2e-3, atol=2e-2)
    assert torch.allclose(cb.float(), pre, rtol=1e-2, atol=0.1)
    assert torch.allclose(s, cb.float().sum(0), rtol=1e-3, atol=0.5)
    assert torch.allclose(s2, (cb.float() ** 2).sum(0), rtol=1e-3, atol=5.0)


@pytest.mark.parametrize("M,N", [(1000, 1000), (130, 72), (802816 // 16, 256), (777, 2048)])
def test_gemm_stats_tails_and_many_tiles(M, N):
    from eagersgd_b200.ops.gemm import gemm, check_error
    torch.manual_seed(M)
    a, b = _rand((M, 64)), _rand((N, 64))
    s = torch.zeros(N, device=DEV)
    s2 = torch.zeros(N, device=DEV)
    c = gemm(a, b, col_sum=s, col_sqsum=s2)
    torch.cuda.synchronize()
    check_error(a.device)
    ref = _ref(a, b, True, True)
    assert torch.allclose(c.float(), ref, rtol=2e-2, atol=0.1)
    assert torch.allclose(s, c.float().sum(0), rtol=2e-3, atol=1.0)
    assert torch.allclose(s2, (c.float() ** 2).sum(0), rtol=2e-3, atol=10.0)


@pytest.mark.parametrize("a_k,b_k", [(True, True), (True, False), (False, True)])
@pytest.mark.parametrize("M,N,K,stats", [(40000, 256, 64, False), (40000, 64, 256, True), (45000, 128, 320, False),
                                         (80000, 512, 128, True), (39000, 200, 136, False)])
def test_gemm_resident_b_operand(M, N, K, stats, a_k, b_k):
    """Long-M, short-K problems keep B in shared memory for all tiles of a CTA: same results as the
    fp32 product, for every operand storage order, with and without the statistics epilogue."""
    from eagersgd_b200.ops.gemm import gemm, check_error
    torch.manual_seed(M + N + K)
    a = _rand((M, K) if a_k else (K, M), 0.5)
    b = _rand((N, K) if b_k else (K, N), 0.5)
    s = torch.zeros(N, device=DEV) if stats else None
    s2 = torch.zeros(N, device=DEV) if stats else None
    c = gemm(a, b, a_kmajor=a_k, b_kmajor=b_k, col_sum=s, col_sqsum=s2)
    torch.cuda.synchronize()
    check_error(a.device)
    ref = _ref(a, b, a_k, b_k)
    assert (c.float() - ref).abs().max().item() <= 0.02 * ref.abs().max().item() + 1e-2
    if stats:
        assert torch.allclose(s, c.float().sum(0), rtol=2e-3, atol=2.0)
        assert torch.allclose(s2, (c.float() ** 2).sum(0), rtol=2e-3, atol=20.0)


@pytest.mark.parametrize("M,N,K", [(300, 72, 64), (4096, 256, 512), (40000, 256, 64), (1000, 520, 96)])
def test_gemm_residual_added_before_rounding(M, N, K):
    from eagersgd_b200.ops.gemm import gemm, check_error
    torch.manual_seed(M + N)
    a, b = _rand((M, K), 0.5), _rand((K, N), 0.5)
    res = _rand((M, N), 2.0)
    c = gemm(a, b, b_kmajor=False, residual=res)
    torch.cuda.synchronize()
    check_error(a.device)
    ref = a.float() @ b.float() + res.float()
    assert (c.float() - ref).abs().max().item() <= 0.01 * ref.abs().max().item() + 1e-2
    # one rounding: closer to the fp32 sum than rounding the product and the sum separately
    two = (gemm(a, b, b_kmajor=False) + res).float()
    assert (c.float() - ref).abs().mean().item() <= (two - ref).abs().mean().item() + 1e-6
