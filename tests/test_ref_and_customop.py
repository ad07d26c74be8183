"""CPU oracles (NumPy and C++) against PyTorch, the operator JIT pipeline, and the validation harness."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from eagersgd_b200.ref import numpy_ops as R
from eagersgd_b200.ref import cpp_ops as CPP


@pytest.mark.parametrize("stride,pad,k", [(1, 1, 3), (2, 1, 3), (2, 3, 7), (1, 0, 1)])
def test_conv_oracles(stride, pad, k):
    rng = np.random.RandomState(0)
    x, w = rng.randn(2, 3, 9, 10).astype(np.float32), rng.randn(4, 3, k, k).astype(np.float32)
    xt, wt = torch.tensor(x, requires_grad=True), torch.tensor(w, requires_grad=True)
    yt = F.conv2d(xt, wt, None, stride, pad)
    dy = rng.randn(*yt.shape).astype(np.float32)
    yt.backward(torch.tensor(dy))
    assert np.allclose(R.conv2d(x, w, stride, pad), yt.detach().numpy(), atol=1e-4)
    assert np.allclose(CPP.conv2d(x, w, stride, pad), yt.detach().numpy(), atol=1e-4)
    for dx, dw in (R.conv2d_grad(x, w, dy.astype(np.float64), stride, pad), CPP.conv2d_grads(x, w, dy, stride, pad)):
        assert np.allclose(dx, xt.grad.numpy(), atol=1e-3) and np.allclose(dw, wt.grad.numpy(), atol=1e-3)


def test_batchnorm_oracles():
    rng = np.random.RandomState(1)
    x = rng.randn(4, 6, 5, 5).astype(np.float32)
    g, b = rng.rand(6).astype(np.float32) + 0.5, rng.randn(6).astype(np.float32)
    xt = torch.tensor(x, requires_grad=True)
    gt, bt = torch.tensor(g, requires_grad=True), torch.tensor(b, requires_grad=True)
    rm, rv = torch.zeros(6), torch.ones(6)
    yt = F.batch_norm(xt, rm, rv, gt, bt, True, 0.1, 1e-5)
    dy = rng.randn(*x.shape).astype(np.float32)
    yt.backward(torch.tensor(dy))
    for mod in (R, CPP):
        y, nrm, nrv, mean, invstd = mod.batchnorm_training(x, g, b, np.zeros(6, np.float32), np.ones(6, np.float32), 0.1)
        assert np.allclose(y, yt.detach().numpy(), atol=1e-4)
        assert np.allclose(nrm, rm.numpy(), atol=1e-5) and np.allclose(nrv, rv.numpy(), atol=1e-4)
        dx, dg, db = mod.batchnorm_training_grad(x, g, mean, invstd, dy)
        assert np.allclose(dx, xt.grad.numpy(), atol=1e-3)
        assert np.allclose(dg, gt.grad.numpy(), atol=1e-3) and np.allclose(db, bt.grad.numpy(), atol=1e-3)


def test_misc_oracles():
    rng = np.random.RandomState(2)
    a, b = rng.randn(5, 7).astype(np.float32), rng.randn(7, 3).astype(np.float32)
    assert np.allclose(CPP.gemm(a, b), a @ b, atol=1e-4)
    assert np.allclose(CPP.gemm(a.T.copy(), b.T.copy(), trans_a=True, trans_b=True), a @ b, atol=1e-4)
    assert np.allclose(R.gemm(a, b, np.ones((5, 3)), 2.0, 0.5), 2 * (a @ b) + 0.5)
    x = rng.randn(2, 3, 8, 8).astype(np.float32)
    t = torch.tensor(x)
    assert np.allclose(R.maxpool(x), F.max_pool2d(t, 3, 2, 1).numpy()) and np.allclose(CPP.maxpool(x), R.maxpool(x))
    assert np.allclose(R.globalaveragepool(x), CPP.global_avgpool(x), atol=1e-5)
    assert np.allclose(R.relu(x), CPP.relu(x))
    logits, labels = rng.randn(6, 10).astype(np.float32), rng.randint(0, 10, 6)
    lt = torch.tensor(logits, requires_grad=True)
    F.cross_entropy(lt, torch.tensor(labels)).backward()
    loss, grad = R.softmax_cross_entropy(logits, labels)
    assert abs(loss - F.cross_entropy(torch.tensor(logits), torch.tensor(labels)).item()) < 1e-5
    assert np.allclose(grad, lt.grad.numpy(), atol=1e-6) and np.allclose(CPP.softmax(logits), R.softmax(logits), atol=1e-6)
    w, acc = R.momentum_sgd(np.ones(3), np.ones(3), np.zeros(3), 0.1, 0.9)
    assert np.allclose(w, 0.9) and np.allclose(acc, 1.0)


SCALE_OP = r'''
#include <eagersgd/op.h>
// y = a * x + b, with gradients for x and b
class ScaleShift : public eagersgd::CustomOperator {
  int64_t n;
 public:
  ScaleShift(const eagersgd::tensor_t* in, int, const eagersgd::tensor_t*, int) : n(in[0].numel()) {}
  void forward(void** in, void** out) override {
    const float* x = (const float*)in[0]; const float* b = (const float*)in[1]; float* y = (float*)out[0];
    for (int64_t i = 0; i < n; ++i) y[i] = SCALE * x[i] + b[i];
  }
  void backward(void** g, void**, void**, void** ig) override {
    const float* dy = (const float*)g[0]; float* dx = (float*)ig[0]; float* db = (float*)ig[1];
    for (int64_t i = 0; i < n; ++i) { dx[i] = SCALE * dy[i]; db[i] = dy[i]; }
  }
  int64_t report(void*) override { return n * 4; }
};
ESGD_REGISTER_OP(ScaleShift)
'''


def test_inline_cpp_operator_and_validation(tmp_path):
    from eagersgd_b200.ops.compile import TensorDescriptor, compile_custom_op, custom_op, custom_python_op
    from eagersgd_b200.ops.validation import test_op_forward, test_op_gradient
    d = TensorDescriptor(torch.float32, (3, 4))
    op = compile_custom_op("scaleshift", SCALE_OP, [d, d], [d], defines={"SCALE": "2.5f"}, output_dir=str(tmp_path))
    fn = custom_op(op)
    x, b = torch.randn(3, 4), torch.randn(3, 4)
    test_op_forward(fn, [x, b], 2.5 * x + b)
    test_op_gradient(fn, [x, b], eps=1e-2, rtol=1e-2, atol=1e-2)
    assert op.report() == 48 and not op.supports_cuda
    sq = custom_python_op(lambda t: t * t, lambda g, ins, outs: (2 * ins[0] * g[0],))
    test_op_gradient(sq, [torch.randn(5)], eps=1e-3, rtol=1e-2, atol=1e-2)
    with pytest.raises(AssertionError):
        bad = custom_python_op(lambda t: t * t, lambda g, ins, outs: (ins[0] * g[0],))
        test_op_gradient(bad, [torch.randn(5) + 2], eps=1e-3)


def test_cpp_oracles_with_backward_match_autograd():
    """Every C++ oracle added for parity with the reference's operator set, forward and backward, against
    PyTorch autograd in double precision."""
    import numpy as np
    import torch
    import torch.nn.functional as F
    from eagersgd_b200.ref import cpp_ops as R
    rng = np.random.RandomState(0)
    t = lambda a: torch.tensor(a, dtype=torch.float64, requires_grad=True)
    close = lambda a, b: np.allclose(a, b.detach().numpy() if hasattr(b, "detach") else b, rtol=1e-4, atol=1e-5)

    a, b = rng.randn(3, 5).astype(np.float32), rng.randn(3, 5).astype(np.float32)
    assert close(R.add(a, b), a + b) and all(close(g, np.ones_like(a) * 2) for g in R.add_grad(np.full_like(a, 2)))
    assert close(R.sum_n([a, b, a]), a + b + a) and len(R.sum_n_grad(a, 3)) == 3
    assert close(R.reshape(a, (5, 3)), a.reshape(5, 3)) and close(R.reshape_grad(a.reshape(5, 3), (3, 5)), a)
    assert close(R.relu_grad(a, b), b * (a > 0))

    A, B, dY = rng.randn(4, 6).astype(np.float32), rng.randn(6, 3).astype(np.float32), rng.randn(4, 3).astype(np.float32)
    ta, tb = t(A), t(B)
    (ta @ tb).backward(torch.tensor(dY, dtype=torch.float64))
    assert close(R.matmul(A, B), A @ B)
    da, db = R.matmul_grad(A, B, dY)
    assert close(da, ta.grad) and close(db, tb.grad)
    for trans_a in (False, True):
        for trans_b in (False, True):
            Ag = rng.randn(6, 4).astype(np.float32) if trans_a else A
            Bg = rng.randn(3, 6).astype(np.float32) if trans_b else B
            ta, tb = t(Ag), t(Bg)
            y = 0.5 * (ta.t() if trans_a else ta) @ (tb.t() if trans_b else tb)
            y.backward(torch.tensor(dY, dtype=torch.float64))
            da, db, dc = R.gemm_grad(Ag, Bg, dY, alpha=0.5, beta=2.0, trans_a=trans_a, trans_b=trans_b)
            assert close(da, ta.grad) and close(db, tb.grad) and close(dc, 2.0 * dY)

    x = rng.randn(5, 7).astype(np.float32)
    tx = t(x)
    ty = torch.softmax(tx, 1)
    g = rng.randn(5, 7).astype(np.float32)
    ty.backward(torch.tensor(g, dtype=torch.float64))
    assert close(R.softmax_grad(R.softmax(x), g), tx.grad)

    x4 = rng.randn(2, 3, 7, 6).astype(np.float32)
    for k, s, p in ((3, 2, 1), (2, 2, 0), (3, 1, 1)):
        tx = t(x4)
        y = F.max_pool2d(tx, k, s, p)
        g = rng.randn(*y.shape).astype(np.float32)
        y.backward(torch.tensor(g, dtype=torch.float64))
        assert close(R.maxpool(x4, k, s, p), y) and close(R.maxpool_grad(x4, g, k, s, p), tx.grad)
        for inc in (False, True):
            tx = t(x4)
            y = F.avg_pool2d(tx, k, s, p, count_include_pad=inc)
            y.backward(torch.tensor(g, dtype=torch.float64))
            assert close(R.avgpool(x4, k, s, p, inc), y) and close(R.avgpool_grad(g, x4.shape, k, s, p, inc), tx.grad)
    tx = t(x4)
    y = tx.mean((2, 3))
    g = rng.randn(2, 3).astype(np.float32)
    y.backward(torch.tensor(g, dtype=torch.float64))
    assert close(R.global_avgpool_grad(g, x4.shape), tx.grad)

    gamma, beta = rng.rand(3).astype(np.float32) + 0.5, rng.randn(3).astype(np.float32)
    mean, var = rng.randn(3).astype(np.float32), rng.rand(3).astype(np.float32) + 0.1
    tx, tg, tb2 = t(x4), t(gamma), t(beta)
    y = F.batch_norm(tx, torch.tensor(mean, dtype=torch.float64), torch.tensor(var, dtype=torch.float64), tg, tb2, False, 0.0, 1e-5)
    g = rng.randn(*x4.shape).astype(np.float32)
    y.backward(torch.tensor(g, dtype=torch.float64))
    assert close(R.batchnorm_inference(x4, gamma, beta, mean, var), y)
    dx, dg, db = R.batchnorm_inference_grad(x4, gamma, mean, var, g)
    assert close(dx, tx.grad) and close(dg, tg.grad) and close(db, tb2.grad)


def test_cpp_oracles_against_autograd_on_random_geometries():
    """Property test of the C++ oracles the GPU kernels are checked against: convolution (forward, data and weight
    gradient), max pooling, average pooling and GEMM with random sizes, strides, paddings and transpositions agree
    with PyTorch's fp32 operators and their autograd."""
    import torch
    import torch.nn.functional as F
    from hypothesis import HealthCheck, given, settings
    from hypothesis import strategies as st
    from eagersgd_b200.ref import cpp_ops as R

    close = lambda a, b: np.allclose(a, b, rtol=2e-4, atol=2e-4)

    @settings(max_examples=40, deadline=None, suppress_health_check=[HealthCheck.too_slow])
    @given(n=st.integers(1, 3), cin=st.integers(1, 5), cout=st.integers(1, 5), h=st.integers(3, 9), w=st.integers(3, 9),
           k=st.sampled_from([1, 2, 3, 5]), stride=st.integers(1, 3), pad=st.integers(0, 2), seed=st.integers(0, 10 ** 6))
    def conv(n, cin, cout, h, w, k, stride, pad, seed):
        if h + 2 * pad < k or w + 2 * pad < k or pad >= k:
            return
        g = torch.Generator().manual_seed(seed)
        x = torch.randn(n, cin, h, w, generator=g, requires_grad=True)
        wt = torch.randn(cout, cin, k, k, generator=g, requires_grad=True)
        y = F.conv2d(x, wt, None, stride, pad)
        dy = torch.randn(y.shape, generator=g)
        y.backward(dy)
        assert close(R.conv2d(x.detach().numpy(), wt.detach().numpy(), stride, pad), y.detach().numpy())
        dx, dw = R.conv2d_grads(x.detach().numpy(), wt.detach().numpy(), dy.numpy(), stride, pad)
        assert close(dx, x.grad.numpy()) and close(dw, wt.grad.numpy())

    @settings(max_examples=40, deadline=None, suppress_health_check=[HealthCheck.too_slow])
    @given(n=st.integers(1, 3), c=st.integers(1, 4), h=st.integers(4, 10), w=st.integers(4, 10), k=st.sampled_from([2, 3]),
           stride=st.integers(1, 3), pad=st.integers(0, 1), seed=st.integers(0, 10 ** 6), include=st.booleans())
    def pools(n, c, h, w, k, stride, pad, seed, include):
        g = torch.Generator().manual_seed(seed)
        x = torch.randn(n, c, h, w, generator=g, requires_grad=True)
        y = F.max_pool2d(x, k, stride, pad)
        dy = torch.randn(y.shape, generator=g)
        y.backward(dy)
        assert close(R.maxpool(x.detach().numpy(), k, stride, pad), y.detach().numpy())
        assert close(R.maxpool_grad(x.detach().numpy(), dy.numpy(), k, stride, pad), x.grad.numpy())
        x.grad = None
        y = F.avg_pool2d(x, k, stride, pad, count_include_pad=include)
        dy = torch.randn(y.shape, generator=g)
        y.backward(dy)
        assert close(R.avgpool(x.detach().numpy(), k, stride, pad, include), y.detach().numpy())
        assert close(R.avgpool_grad(dy.numpy(), tuple(x.shape), k, stride, pad, include), x.grad.numpy())

    @settings(max_examples=40, deadline=None, suppress_health_check=[HealthCheck.too_slow])
    @given(m=st.integers(1, 7), n=st.integers(1, 7), kk=st.integers(1, 7), ta=st.booleans(), tb=st.booleans(),
           alpha=st.sampled_from([1.0, 0.5, -2.0]), beta=st.sampled_from([0.0, 1.0, 0.25]), seed=st.integers(0, 10 ** 6))
    def gemm(m, n, kk, ta, tb, alpha, beta, seed):
        g = torch.Generator().manual_seed(seed)
        a = torch.randn((kk, m) if ta else (m, kk), generator=g)
        b = torch.randn((n, kk) if tb else (kk, n), generator=g)
        c = torch.randn(m, n, generator=g)
        want = alpha * ((a.t() if ta else a) @ (b.t() if tb else b)) + beta * c
        assert close(R.gemm(a.numpy(), b.numpy(), c.numpy(), alpha, beta, ta, tb), want.numpy())

    conv()
    pools()
    gemm()
