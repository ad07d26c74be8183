"""The graph executor's operators beyond the ResNet set, each against a direct PyTorch / numpy computation of the
ONNX semantics (the reference tests its visitors with the ONNX backend test data: deep500/utils/onnx_interop/
onnx_test_parser.py, samples/onnxtest.py)."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from eagersgd_b200.graph import Graph, GraphNetwork


def _run(op_type, inputs, n_out=1, **attrs):
    """inputs: list of (name, value, is_initializer); the first non-initializer is the graph input."""
    g = Graph("t")
    names, feeds, first = [], {}, None
    for name, value, is_init in inputs:
        names.append(name)
        if is_init:
            g.add_initializer(name, np.asarray(value))
        else:
            g.add_input(name)
            if first is None:
                first = (name, value)
            else:
                feeds[name] = value
    g.add_initializer("_dummy", np.zeros(1, np.float32))           # the executor asks a parameter for its device
    outs = ["y%d" % i for i in range(n_out)]
    g.add(op_type, names, outs, **attrs)
    for o in outs:
        g.add_output(o)
    res = GraphNetwork(g, trainable_only_used=False)(first[1], **feeds)
    return res


X = torch.tensor([[-1.5, 0.0, 2.5, -0.25], [3.0, -2.0, 0.5, 1.0]])
Y = torch.tensor([[1.0, 0.0, -2.5, 4.0], [3.0, 2.0, 0.25, -1.0]])
I64 = lambda *v: np.asarray(v, dtype=np.int64)


@pytest.mark.parametrize("op,ref", [
    ("Floor", torch.floor), ("Ceil", torch.ceil), ("Round", torch.round), ("Sign", torch.sign), ("Erf", torch.erf),
    ("Sin", torch.sin), ("Cos", torch.cos), ("Softplus", F.softplus), ("Softsign", F.softsign), ("Elu", F.elu),
    ("Selu", F.selu), ("HardSigmoid", lambda x: (0.2 * x + 0.5).clamp(0, 1)), ("IsNaN", torch.isnan),
    ("ThresholdedRelu", lambda x: torch.where(x > 1.0, x, torch.zeros_like(x))),
    ("Reciprocal", lambda x: 1.0 / x),
])
def test_unary_operators(op, ref):
    x = X + 0.125 if op == "Reciprocal" else X
    got = _run(op, [("x", x, False)])
    assert torch.allclose(got.float(), ref(x).float(), atol=1e-6), op


@pytest.mark.parametrize("op,ref", [
    ("Equal", torch.eq), ("Greater", torch.gt), ("GreaterOrEqual", torch.ge), ("Less", torch.lt), ("LessOrEqual", torch.le),
    ("Max", torch.maximum), ("Min", torch.minimum), ("Mean", lambda a, b: (a + b) / 2), ("PRelu", lambda a, b: torch.where(a >= 0, a, a * b)),
])
def test_binary_operators(op, ref):
    got = _run(op, [("a", X, False), ("b", Y, False)])
    assert torch.equal(got, ref(X, Y)) if got.dtype == torch.bool else torch.allclose(got, ref(X, Y)), op


def test_logic_where_and_cast():
    a, b = X > 0, Y > 0
    assert torch.equal(_run("And", [("a", a, False), ("b", b, False)]), a & b)
    assert torch.equal(_run("Or", [("a", a, False), ("b", b, False)]), a | b)
    assert torch.equal(_run("Xor", [("a", a, False), ("b", b, False)]), a ^ b)
    assert torch.equal(_run("Not", [("a", a, False)]), ~a)
    assert torch.equal(_run("Where", [("c", a, False), ("p", X, False), ("q", Y, False)]), torch.where(a, X, Y))
    assert _run("Cast", [("x", X, False)], to=7).dtype == torch.int64


@pytest.mark.parametrize("op,ref", [
    ("ReduceMax", lambda x: x.amax(1, keepdim=True)), ("ReduceMin", lambda x: x.amin(1, keepdim=True)),
    ("ReduceProd", lambda x: x.prod(1, keepdim=True)), ("ReduceL1", lambda x: x.abs().sum(1, keepdim=True)),
    ("ReduceL2", lambda x: x.square().sum(1, keepdim=True).sqrt()), ("ReduceSumSquare", lambda x: x.square().sum(1, keepdim=True)),
    ("ReduceLogSumExp", lambda x: torch.logsumexp(x, 1, keepdim=True)), ("ReduceMean", lambda x: x.mean(1, keepdim=True)),
])
def test_reductions_with_axes_as_attribute_and_as_input(op, ref):
    assert torch.allclose(_run(op, [("x", X, False)], axes=[1]), ref(X), atol=1e-6)
    if op in ("ReduceMean",):
        return
    flat = _run(op, [("x", X, False)], keepdims=0)                         # no axes: over everything
    assert flat.dim() == 0
    assert torch.allclose(_run("ReduceSum", [("x", X, False), ("axes", I64(0), True)], keepdims=0), X.sum(0))


def test_arg_topk_cumsum():
    assert torch.equal(_run("ArgMax", [("x", X, False)], axis=1, keepdims=0), X.argmax(1))
    assert torch.equal(_run("ArgMin", [("x", X, False)], axis=0), X.argmin(0, keepdim=True))
    v, i = _run("TopK", [("x", X, False), ("k", I64(2), True)], n_out=2, axis=1)
    tv, ti = torch.topk(X, 2, dim=1)
    assert torch.equal(v, tv) and torch.equal(i, ti)
    assert torch.allclose(_run("CumSum", [("x", X, False), ("axis", I64(1), True)]), X.cumsum(1))
    want = (X.flip(1).cumsum(1) - X.flip(1)).flip(1)
    assert torch.allclose(_run("CumSum", [("x", X, False), ("axis", I64(1), True)], reverse=1, exclusive=1), want)


def test_shape_and_data_movement():
    x = torch.arange(24.0).reshape(2, 3, 4)
    assert _run("Shape", [("x", x, False)]).tolist() == [2, 3, 4] and int(_run("Size", [("x", x, False)])) == 24
    assert torch.equal(_run("Reshape", [("x", x, False), ("s", I64(0, -1), True)]), x.reshape(2, 12))
    assert torch.equal(_run("Expand", [("x", x[:, :1], False), ("s", I64(2, 3, 4), True)]), x[:, :1].expand(2, 3, 4))
    assert torch.equal(_run("Tile", [("x", x, False), ("r", I64(1, 2, 1), True)]), x.repeat(1, 2, 1))
    assert torch.equal(_run("Gather", [("x", x, False), ("i", I64([0, 2], [1, -1]), True)], axis=1), x[:, [[0, 2], [1, 2]]])
    got = _run("Slice", [("x", x, False), ("st", I64(1, 0), True), ("en", I64(3, -1), True), ("ax", I64(1, 2), True), ("sp", I64(1, 2), True)])
    assert torch.equal(got, x[:, 1:3, 0:-1:2])
    a, b = _run("Split", [("x", x, False), ("s", I64(1, 3), True)], n_out=2, axis=2)
    assert torch.equal(a, x[:, :, :1]) and torch.equal(b, x[:, :, 1:])
    assert torch.equal(_run("Squeeze", [("x", x[:, :1], False), ("a", I64(1), True)]), x[:, 0])
    assert _run("Unsqueeze", [("x", x, False), ("a", I64(0, 4), True)]).shape == (1, 2, 3, 4, 1)
    assert torch.equal(_run("ConstantOfShape", [("s", torch.tensor([2, 2]), False)], value=np.asarray([7], np.int64)),
                       torch.full((2, 2), 7))
    img = torch.arange(32.0).reshape(1, 8, 2, 2)
    d2s = _run("DepthToSpace", [("x", img, False)], blocksize=2)
    assert torch.equal(d2s, F.pixel_shuffle(img.reshape(1, 2, 2, 2, 2, 2).permute(0, 3, 1, 2, 4, 5).reshape(1, 8, 2, 2), 2))
    assert torch.equal(_run("DepthToSpace", [("x", img, False)], blocksize=2, mode="CRD"), F.pixel_shuffle(img, 2))
    assert torch.equal(_run("SpaceToDepth", [("x", d2s, False)], blocksize=2), img)      # the inverse of the DCR form
    hot = _run("OneHot", [("i", torch.tensor([0, 2]), False), ("d", I64(3), True), ("v", np.asarray([0.0, 5.0], np.float32), True)])
    assert hot.tolist() == [[5.0, 0.0, 0.0], [0.0, 0.0, 5.0]]


def test_layers():
    torch.manual_seed(0)
    x, w, b = torch.randn(2, 4, 5, 5), torch.randn(4, 3, 3, 3), torch.randn(3)
    got = _run("ConvTranspose", [("x", x, False), ("w", w.numpy(), True), ("b", b.numpy(), True)], strides=[2, 2],
               pads=[1, 1, 1, 1], output_padding=[1, 1])
    assert torch.allclose(got, F.conv_transpose2d(x, w, b, stride=2, padding=1, output_padding=1), atol=1e-5)
    s, t = torch.rand(4) + 0.5, torch.randn(4)
    got = _run("InstanceNormalization", [("x", x, False), ("s", s.numpy(), True), ("t", t.numpy(), True)], epsilon=1e-5)
    assert torch.allclose(got, F.instance_norm(x, weight=s, bias=t, eps=1e-5), atol=1e-5)
    assert torch.equal(_run("GlobalMaxPool", [("x", x, False)]), x.amax((2, 3), keepdim=True))
    assert torch.allclose(_run("LpNormalization", [("x", x, False)], axis=1, p=2), x / x.norm(dim=1, keepdim=True), atol=1e-6)
    up = _run("Resize", [("x", x, False), ("roi", np.zeros(0, np.float32), True), ("sc", np.asarray([1, 1, 2, 2], np.float32), True)])
    assert torch.equal(up, F.interpolate(x, scale_factor=2.0, mode="nearest"))
    up = _run("Upsample", [("x", x, False), ("sc", np.asarray([1, 1, 2, 2], np.float32), True)])
    assert up.shape == (2, 4, 10, 10)


def test_onnx_lstm_runs_on_the_lstm_layer():
    """An ONNX LSTM node (gates ordered i, o, f, c; split bias) against torch.nn.LSTM with the same weights."""
    torch.manual_seed(1)
    T, B, I, H = 5, 3, 8, 16
    ref = torch.nn.LSTM(I, H)
    x = torch.randn(T, B, I)
    to_onnx = torch.cat([torch.arange(0, H), torch.arange(3 * H, 4 * H), torch.arange(H, 2 * H), torch.arange(2 * H, 3 * H)])
    w = ref.weight_ih_l0.detach()[to_onnx].unsqueeze(0).numpy()
    r = ref.weight_hh_l0.detach()[to_onnx].unsqueeze(0).numpy()
    b = torch.cat([ref.bias_ih_l0.detach()[to_onnx], ref.bias_hh_l0.detach()[to_onnx]]).unsqueeze(0).numpy()
    y, y_h = _run("LSTM", [("x", x, False), ("w", w, True), ("r", r, True), ("b", b, True)], n_out=2, hidden_size=H)
    want, (h_n, _) = ref(x)
    assert y.shape == (T, 1, B, H) and torch.allclose(y[:, 0], want, atol=1e-5)
    assert torch.allclose(y_h, h_n, atol=1e-5)


def test_experimental_operators_of_early_onnx():
    """Affine, Scale, ScaledTanh, ParametricSoftplus, ImageScaler, Crop, ConstantFill, GivenTensorFill: the operator
    classes the reference generated from its ONNX release (deep500/utils/onnx_interop/generated_operators.py)."""
    from eagersgd_b200.graph import onnx_ops
    for name in ("ATen", "Affine", "ConstantFill", "Crop", "GRUUnit", "GivenTensorFill", "ImageScaler", "LoopIndexTensor",
                 "ParametricSoftplus", "Scale", "ScaledTanh"):
        assert onnx_ops.operator_class(name) is not None, name
    assert torch.allclose(_run("Affine", [("x", X, False)], alpha=2.0, beta=-1.0), 2 * X - 1)
    assert torch.allclose(_run("Scale", [("x", X, False)], scale=0.5), X / 2)
    assert torch.allclose(_run("ScaledTanh", [("x", X, False)], alpha=1.5, beta=0.5), 1.5 * torch.tanh(0.5 * X))
    assert torch.allclose(_run("ParametricSoftplus", [("x", X, False)], alpha=2.0, beta=3.0), 2 * torch.log(torch.exp(3 * X) + 1),
                          atol=1e-6)
    img = torch.arange(2 * 3 * 4 * 5, dtype=torch.float32).reshape(2, 3, 4, 5)
    got = _run("ImageScaler", [("x", img, False)], scale=0.1, bias=[1.0, 2.0, 3.0])
    assert torch.allclose(got, img * 0.1 + torch.tensor([1.0, 2.0, 3.0]).view(1, 3, 1, 1))
    assert torch.equal(_run("Crop", [("x", img, False)], border=[1, 0, 2, 1]), img[:, :, 0:3, 1:3])
    assert torch.equal(_run("Crop", [("x", img, False)], border=[1, 1, 0, 0], scale=[2, 3]), img[:, :, 1:3, 1:4])
    got = _run("ConstantFill", [("x", X, False)], value=2.5)
    assert got.shape == X.shape and torch.all(got == 2.5)
    got = _run("ConstantFill", [("s", I64(2, 3), False)], input_as_shape=1, extra_shape=[4], value=7, dtype=7)
    assert got.shape == (2, 3, 4) and got.dtype == torch.int64 and torch.all(got == 7)
    got = _run("GivenTensorFill", [("x", torch.zeros(2, 2), False)], values=[1.0, 2.0, 3.0, 4.0])
    assert torch.equal(got, torch.tensor([[1.0, 2.0], [3.0, 4.0]]))
    op = onnx_ops.make_operation("ATen", ["a", "b"], ["c"], operator="index_select", dim=1)      # any attribute is allowed
    op.validate()
    with pytest.raises(ValueError, match="no attribute"):
        onnx_ops.make_operation("Affine", ["a"], ["b"], gamma=1.0).validate()
