import numpy as np
import pytest
import torch

from eagersgd_b200.graph import Graph, GraphNetwork, OpCounter, from_torch_resnet
from eagersgd_b200.models.resnet import cifar_resnet


def test_resnet_graph_matches_module(tmp_path):
    torch.manual_seed(0)
    m = cifar_resnet(8).eval()
    for mod in m.modules():
        if isinstance(mod, torch.nn.BatchNorm2d):
            torch.nn.init.uniform_(mod.weight, 0.5, 1.0)
            mod.running_mean.normal_(0, 0.1)
    g = from_torch_resnet(m)
    counts = g.accept(OpCounter())
    assert counts["Conv"] == counts["BatchNormalization"] >= 7 and counts["Gemm"] == 1 and counts["Add"] == 3
    net = GraphNetwork(g).eval()
    x = torch.randn(2, 3, 32, 32)
    assert torch.allclose(net(x), m(x), atol=1e-4)
    g.save(str(tmp_path / "resnet8"))
    g2 = Graph.load(str(tmp_path / "resnet8"))
    assert torch.allclose(GraphNetwork(g2).eval()(x), m(x), atol=1e-4)
    assert g.to_dot().startswith("digraph")


def test_graph_training_with_loss_and_extensions():
    from eagersgd_b200.train.executor import GraphExecutor
    rng = np.random.RandomState(0)
    g = Graph("mlp")
    g.add_input("x")
    g.add_initializer("w1", rng.randn(16, 8).astype(np.float32) * 0.3)
    g.add_initializer("b1", np.zeros(16, np.float32))
    g.add_initializer("w2", rng.randn(4, 16).astype(np.float32) * 0.3)
    g.add_initializer("b2", np.zeros(4, np.float32))
    g.add("Gemm", ["x", "w1", "b1"], ["h"], transB=1)
    g.add("Relu", ["h"], ["hr"])
    g.add("AllReduceGradients", ["hr"], ["hs"])      # identity forward, averages the gradient (world 1: no-op)
    g.add("Gemm", ["hs", "w2", "b2"], ["logits"], transB=1)
    g.add_output("logits")
    net = GraphNetwork(g)
    assert len(list(net.parameters())) == 4
    x = torch.randn(64, 8)
    y = (x[:, 0] > 0).long() + 2 * (x[:, 1] > 0).long()
    opt = torch.optim.SGD(net.parameters(), lr=0.5)
    first = None
    for _ in range(60):
        opt.zero_grad()
        loss = torch.nn.functional.cross_entropy(net(x), y)
        loss.backward()
        opt.step()
        first = first or loss.item()
    assert loss.item() < 0.5 * first
    g.add_loss("SoftmaxCrossEntropy", "logits")
    net2 = GraphNetwork(g)
    logits, l2 = net2(x, label=y)
    assert l2.dim() == 0 and logits.shape == (64, 4)
    g.add("StopGradient", ["logits"], ["frozen"])
    g.add_output("frozen")
    outs = GraphNetwork(g)(x, label=y)
    assert not outs[-1].requires_grad


def test_elementwise_and_shape_operators():
    import torch.nn.functional as F
    g = Graph("misc")
    g.add_input("x")
    g.add_initializer("w", np.full((1, 3, 1, 1), 2.0, np.float32))
    g.add("Mul", ["x", "w"], ["a"])
    g.add("Constant", [], ["one"], value=[[[[1.0]]]])
    g.add("Sub", ["a", "one"], ["b"])
    g.add("LeakyRelu", ["b"], ["c"], alpha=0.1)
    g.add("Pad", ["c"], ["d"], pads=[0, 0, 1, 2, 0, 0, 3, 4], value=0.0)
    g.add("ReduceMean", ["d"], ["e"], axes=[2, 3], keepdims=0)
    g.add("Transpose", ["e"], ["f"], perm=[1, 0])
    g.add("Tanh", ["f"], ["h"])
    g.add("Clip", ["h"], ["out"], min=-0.5, max=0.5)
    g.add_output("out")
    from eagersgd_b200.graph import STANDARD_OPS
    assert all(op.op_type in STANDARD_OPS for op in g.ops)
    x = torch.randn(2, 3, 4, 5)
    out = GraphNetwork(g)(x)
    ref = F.pad(F.leaky_relu(x * 2.0 - 1.0, 0.1), [2, 4, 1, 3]).mean((2, 3)).t().tanh().clamp(-0.5, 0.5)
    assert out.shape == (3, 2) and torch.allclose(out, ref, atol=1e-6)


def test_onnx_file_round_trip(tmp_path):
    """A graph written as a .onnx file (protobuf wire format, no onnx package) reads back with the same
    nodes, attributes of every kind, initializers and inputs / outputs."""
    import numpy as np
    from eagersgd_b200.graph.ir import Graph
    from eagersgd_b200.graph.onnx_io import load_onnx, save_onnx
    g = Graph("net")
    g.add_input("x")
    g.add_initializer("w", np.random.randn(4, 3, 3, 3).astype(np.float32))
    g.add_initializer("idx", np.arange(6, dtype=np.int64).reshape(2, 3))
    g.add("Conv", ["x", "w"], ["y"], kernel_shape=[3, 3], pads=[1, 1, 1, 1], strides=[2, 2], group=1, auto_pad="NOTSET")
    g.add("LeakyRelu", ["y"], ["z"], alpha=0.25)
    g.add("Constant", [], ["c"], value=np.array([1.5, -2.0], dtype=np.float32))
    g.add("Pad", ["z"], ["out"], pads=[0, 0, 1, 1, 0, 0, 1, 1], mode="constant", scales=[1.0, 0.5])
    g.add_output("out")
    path = str(tmp_path / "net.onnx")
    save_onnx(g, path)
    h = load_onnx(path)
    assert h.name == "net" and h.inputs == ["x"] and h.outputs == ["out"]
    assert [o.op_type for o in h.ops] == ["Conv", "LeakyRelu", "Constant", "Pad"]
    assert h.ops[0].attrs["pads"] == [1, 1, 1, 1] and h.ops[0].attrs["auto_pad"] == "NOTSET" and h.ops[0].attrs["group"] == 1
    assert abs(h.ops[1].attrs["alpha"] - 0.25) < 1e-7 and h.ops[3].attrs["scales"] == [1.0, 0.5]
    assert np.array_equal(h.ops[2].attrs["value"], np.array([1.5, -2.0], dtype=np.float32))
    assert np.array_equal(h.initializers["w"], g.initializers["w"]) and h.initializers["idx"].dtype == np.int64
    assert h.meta["opsets"][""] == 13


def test_onnx_file_from_the_torch_exporter_runs_on_the_executor(tmp_path):
    """A model exported by PyTorch's own ONNX exporter is parsed and gives the exporter model's outputs."""
    import numpy as np
    import torch
    from eagersgd_b200.graph.executor import GraphNetwork
    from eagersgd_b200.graph.onnx_io import load_onnx
    torch.manual_seed(0)
    m = torch.nn.Sequential(torch.nn.Conv2d(3, 8, 3, padding=1), torch.nn.BatchNorm2d(8), torch.nn.ReLU(),
                            torch.nn.MaxPool2d(2), torch.nn.Flatten(), torch.nn.Linear(8 * 4 * 4, 5)).eval()
    x = torch.randn(2, 3, 8, 8)
    path = str(tmp_path / "m.onnx")
    try:
        torch.onnx.export(m, (x,), path, input_names=["x"], output_names=["y"], opset_version=13, dynamo=False)
    except Exception as e:   # noqa
        pytest.skip("this PyTorch cannot export without extra packages: %s" % str(e)[:80])
    g = load_onnx(path)
    assert g.inputs == ["x"] and g.outputs == ["y"] and any(o.op_type == "Conv" for o in g.ops)
    net = GraphNetwork(g).eval()
    with torch.no_grad():
        got = net(x)
        ref = m(x)
    got = got[0] if isinstance(got, (list, tuple)) else got
    assert torch.allclose(got.float(), ref, rtol=1e-4, atol=1e-4)


def test_resnet_graph_survives_an_onnx_file(tmp_path):
    """Model -> graph -> .onnx file -> graph -> executor: same logits as the model."""
    from eagersgd_b200.graph import load_onnx, save_onnx
    torch.manual_seed(3)
    model = cifar_resnet(8, 1, 10).eval()
    g = from_torch_resnet(model)
    path = str(tmp_path / "resnet8.onnx")
    save_onnx(g, path)
    h = load_onnx(path)
    assert len(h.ops) == len(g.ops) and sorted(h.initializers) == sorted(g.initializers)
    x = torch.randn(2, 3, 32, 32)
    with torch.no_grad():
        a = GraphNetwork(g).eval()(x)
        b = GraphNetwork(h).eval()(x)
    a = a[0] if isinstance(a, (list, tuple)) else a
    b = b[0] if isinstance(b, (list, tuple)) else b
    assert torch.allclose(a, b, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("use_cpp", [True, False])
def test_reference_executor_matches_native_executor(use_cpp):
    """The same ResNet graph on the CPU oracles (numpy / compiled C++) and on the native executor: logits,
    loss and the gradient of every weight agree."""
    from eagersgd_b200.graph import ReferenceGraphExecutor
    torch.manual_seed(4)
    model = cifar_resnet(8, 1, 10).train()
    for m in model.modules():                     # give the zero-initialised gammas a value: every path carries gradient
        if isinstance(m, torch.nn.BatchNorm2d):
            torch.nn.init.uniform_(m.weight, 0.5, 1.5)
    g = from_torch_resnet(model)
    g.add_loss("SoftmaxCrossEntropy", g.outputs[0])
    x = torch.randn(4, 3, 32, 32)
    y = torch.randint(0, 10, (4,))
    net = GraphNetwork(g).train()
    outs = net(x, label=y)
    outs[-1].backward()
    ref = ReferenceGraphExecutor(g, use_cpp=use_cpp)
    r_outs = ref.inference_and_backprop({g.inputs[0]: x.numpy(), "label": y.numpy()})
    assert np.allclose(r_outs[0], outs[0].detach().numpy(), rtol=1e-3, atol=1e-3)
    assert abs(float(r_outs[-1]) - float(outs[-1])) < 1e-3
    checked = 0
    for name in g.get_params():
        p = net.tensor(name)
        if p.grad is None or name not in ref.gradients:
            continue
        a, b = ref.gradients[name], p.grad.numpy()
        assert np.allclose(a, b, rtol=2e-2, atol=2e-3 * max(1.0, float(np.abs(b).max()))), name
        checked += 1
    assert checked >= 20


def test_onnx_operator_classes():
    """Every standard operator has a class with its attributes and defaults; nodes of graphs built in code and of
    parsed files are instances of them; validation names what is wrong."""
    from eagersgd_b200.graph import Graph, operator_class, operator_names
    from eagersgd_b200.graph.ir import Operation
    names = operator_names()
    assert len(names) >= 150 and {"Conv", "BatchNormalization", "LSTM", "Einsum", "Resize", "TopK"} <= set(names)
    g = Graph("t")
    g.add_input("x")
    g.add_initializer("w", np.zeros((4, 3, 3, 3), np.float32))
    conv = g.add("Conv", ["x", "w"], ["y"], kernel_shape=[3, 3], pads=[1, 1, 1, 1])
    assert isinstance(conv, operator_class("Conv")) and isinstance(conv, Operation)
    assert conv.group == 1 and conv.auto_pad == "NOTSET" and conv.pads == [1, 1, 1, 1] and conv.strides is None
    conv.validate()
    pool = g.add("MaxPool", ["y"], ["z"])
    with pytest.raises(ValueError, match="kernel_shape"):
        pool.validate()
    with pytest.raises(AttributeError):
        pool.kernel_shape
    bad = g.add("Relu", ["z", "z"], ["r"], slope=0.1)
    with pytest.raises(ValueError, match="slope"):
        bad.validate()
    bad.attrs.clear()
    with pytest.raises(ValueError, match="inputs"):
        bad.validate()
    custom = g.add("MyOwnOp", ["r"], ["s"], anything=1)
    assert type(custom) is Operation and operator_class("MyOwnOp") is None
    counts = g.accept(OpCounter())                                  # visitor dispatch is unchanged
    assert counts["Conv"] == 1 and counts["MyOwnOp"] == 1
    for n in names:                                                 # every class can be made and validated
        cls = operator_class(n)
        assert cls.__name__ == n and cls.MIN_INPUTS <= cls.MAX_INPUTS


@pytest.mark.parametrize("name,kw,shape", [("simple_mnist", {}, (3, 1, 28, 28)), ("deep_mnist", {}, (2, 1, 28, 28)),
                                           ("wide_resnet", dict(depth=10, widen=1), (2, 3, 32, 32))])
def test_any_traceable_module_becomes_a_graph_and_an_onnx_file(name, kw, shape, tmp_path):
    """``torch.fx`` trace -> model graph -> .onnx file -> graph -> executor: the outputs of the module."""
    from eagersgd_b200.graph import GraphNetwork, export_network, from_torch_module, load_onnx
    from eagersgd_b200.models import create_model
    torch.manual_seed(5)
    m = create_model(name, **kw).eval()
    for mod in m.modules():
        if isinstance(mod, torch.nn.BatchNorm2d):
            mod.running_mean.normal_(0, 0.2)
            mod.running_var.uniform_(0.5, 1.5)
    x = torch.randn(*shape)
    g = from_torch_module(m)
    for op in g.ops:
        if hasattr(op, "validate"):
            op.validate()                                   # every node is a well-formed standard operator
    with torch.no_grad():
        want = m(x)
        got = GraphNetwork(g).eval()(x)
    got = got[0] if isinstance(got, (list, tuple)) else got
    assert torch.allclose(got, want, rtol=1e-4, atol=1e-4)
    path = export_network(m, str(tmp_path / (name + ".onnx")))
    with torch.no_grad():
        again = GraphNetwork(load_onnx(path)).eval()(x)
    again = again[0] if isinstance(again, (list, tuple)) else again
    assert torch.allclose(again, want, rtol=1e-4, atol=1e-4)


def test_untraceable_operations_are_named():
    from eagersgd_b200.graph import from_torch_module

    class Odd(torch.nn.Module):
        def forward(self, x):
            return torch.erf(x)

    with pytest.raises(NotImplementedError, match="erf"):
        from_torch_module(Odd())


def test_onnx_round_trip_of_random_graphs():
    """Property test of the .onnx writer and reader: graphs with random node attributes (negative and large
    integers, floats, unicode strings, lists, tensors of several element types and ranks, empty lists) and random
    initializers come back equal."""
    import tempfile
    from hypothesis import HealthCheck, given, settings
    from hypothesis import strategies as st
    from hypothesis.extra import numpy as hnp
    from eagersgd_b200.graph.ir import Graph
    from eagersgd_b200.graph.onnx_io import load_onnx, save_onnx

    f32 = st.floats(width=32, allow_nan=False, allow_infinity=False)
    i64 = st.integers(min_value=-(1 << 62), max_value=(1 << 62))
    tensors = st.one_of(
        hnp.arrays(np.float32, hnp.array_shapes(min_dims=0, max_dims=3, max_side=4), elements=f32),
        hnp.arrays(np.int64, hnp.array_shapes(min_dims=1, max_dims=2, max_side=5), elements=i64),
        hnp.arrays(np.float64, hnp.array_shapes(min_dims=1, max_dims=2, max_side=3),
                   elements=st.floats(allow_nan=False, allow_infinity=False, width=64)),
        hnp.arrays(np.int32, hnp.array_shapes(min_dims=1, max_dims=2, max_side=4),
                   elements=st.integers(-(1 << 31), (1 << 31) - 1)),
        hnp.arrays(np.uint8, hnp.array_shapes(min_dims=1, max_dims=2, max_side=6), elements=st.integers(0, 255)),
        hnp.arrays(np.bool_, hnp.array_shapes(min_dims=1, max_dims=1, max_side=6)))
    attr = st.one_of(i64, f32, st.text(max_size=12), st.lists(i64, max_size=5), st.lists(f32, min_size=1, max_size=5), tensors)
    names = st.text(alphabet="abcdefghij_", min_size=1, max_size=6)
    attrs = st.dictionaries(names, attr, max_size=4)
    nodes = st.lists(st.tuples(st.sampled_from(["Relu", "Conv", "MyOp", "Add"]), attrs), min_size=1, max_size=4)

    @settings(max_examples=60, deadline=None, suppress_health_check=[HealthCheck.too_slow])
    @given(nodes=nodes, inits=st.lists(tensors, max_size=3))
    def check(nodes, inits):
        g = Graph("g")
        g.add_input("x")
        prev = "x"
        for k, t in enumerate(inits):
            g.add_initializer("w%d" % k, t)
        for k, (op_type, a) in enumerate(nodes):
            out = "t%d" % k
            g.add(op_type, [prev], [out], **a)
            prev = out
        g.add_output(prev)
        with tempfile.TemporaryDirectory() as d:
            path = d + "/g.onnx"
            save_onnx(g, path)
            h = load_onnx(path)
        assert [o.op_type for o in h.ops] == [o.op_type for o in g.ops]
        assert h.inputs == g.inputs and h.outputs == g.outputs
        for a, b in zip(g.ops, h.ops):
            assert a.inputs == b.inputs and a.outputs == b.outputs and set(a.attrs) == set(b.attrs), (a.attrs, b.attrs)
            for key, v in a.attrs.items():
                w = b.attrs[key]
                if isinstance(v, np.ndarray):
                    assert isinstance(w, np.ndarray) and w.dtype == v.dtype and w.shape == v.shape and np.array_equal(w, v), (key, v, w)
                elif isinstance(v, float):
                    assert w == pytest.approx(v, rel=1e-6, abs=1e-38), (key, v, w)
                elif isinstance(v, list) and v and isinstance(v[0], float):
                    assert w == pytest.approx(v, rel=1e-6, abs=1e-38), (key, v, w)
                else:
                    assert w == v, (key, v, w)
        for k, t in enumerate(inits):
            w = h.initializers["w%d" % k]
            assert w.dtype == t.dtype and w.shape == t.shape and np.array_equal(w, t)

    check()


def test_random_sequential_networks_survive_tracing_and_an_onnx_file():
    """Property test: random small convolutional networks (kernel sizes, strides, paddings, biases, normalisation,
    activations, pooling, a dense head) give the same outputs as a graph and after a trip through an .onnx file."""
    import tempfile
    from hypothesis import HealthCheck, given, settings
    from hypothesis import strategies as st
    from eagersgd_b200.graph import GraphNetwork, from_torch_module, load_onnx, save_onnx

    layer = st.one_of(
        st.tuples(st.just("conv"), st.integers(1, 6), st.sampled_from([1, 3]), st.integers(1, 2), st.integers(0, 1), st.booleans()),
        st.tuples(st.just("bn")), st.tuples(st.just("relu")), st.tuples(st.just("leaky"), st.sampled_from([0.01, 0.2])),
        st.tuples(st.just("sigmoid")), st.tuples(st.just("tanh")),
        st.tuples(st.just("maxpool"), st.sampled_from([2, 3]), st.integers(1, 2)),
        st.tuples(st.just("avgpool"), st.sampled_from([2]), st.integers(1, 2)))

    @settings(max_examples=40, deadline=None, suppress_health_check=[HealthCheck.too_slow])
    @given(layers=st.lists(layer, min_size=1, max_size=6), cin=st.integers(1, 3), classes=st.integers(1, 5),
           seed=st.integers(0, 10 ** 6))
    def check(layers, cin, classes, seed):
        torch.manual_seed(seed)
        mods, c, size = [], cin, 12
        for spec in layers:
            kind = spec[0]
            if kind == "conv":
                _, co, k, s, p, bias = spec
                if size + 2 * p < k:
                    continue
                mods.append(torch.nn.Conv2d(c, co, k, s, p, bias=bias))
                c, size = co, (size + 2 * p - k) // s + 1
            elif kind == "bn":
                bn = torch.nn.BatchNorm2d(c)
                bn.running_mean.normal_(0, 0.3)
                bn.running_var.uniform_(0.5, 2.0)
                mods.append(bn)
            elif kind == "relu":
                mods.append(torch.nn.ReLU())
            elif kind == "leaky":
                mods.append(torch.nn.LeakyReLU(spec[1]))
            elif kind == "sigmoid":
                mods.append(torch.nn.Sigmoid())
            elif kind == "tanh":
                mods.append(torch.nn.Tanh())
            elif kind in ("maxpool", "avgpool"):
                _, k, s = spec
                if size < k:
                    continue
                mods.append((torch.nn.MaxPool2d if kind == "maxpool" else torch.nn.AvgPool2d)(k, s))
                size = (size - k) // s + 1
        mods += [torch.nn.Flatten(), torch.nn.Linear(c * size * size, classes)]
        m = torch.nn.Sequential(*mods).eval()
        x = torch.randn(2, cin, 12, 12)
        with torch.no_grad():
            want = m(x)
            g = from_torch_module(m)
            got = GraphNetwork(g).eval()(x)
            with tempfile.TemporaryDirectory() as d:
                save_onnx(g, d + "/m.onnx")
                again = GraphNetwork(load_onnx(d + "/m.onnx")).eval()(x)
        for y in (got, again):
            y = y[0] if isinstance(y, (list, tuple)) else y
            assert torch.allclose(y, want, rtol=1e-4, atol=1e-4), (layers, (y - want).abs().max())

    check()


@pytest.mark.parametrize("use_cpp", [True, False])
def test_reference_executor_gradients_on_random_networks(use_cpp):
    """Property test of the CPU reference executor (numpy and compiled C++ operators, forward and backward): on
    random small networks with a softmax-cross-entropy loss its logits, loss and every weight gradient agree with
    the native executor's autograd."""
    from hypothesis import HealthCheck, given, settings
    from hypothesis import strategies as st
    from eagersgd_b200.graph import GraphNetwork, ReferenceGraphExecutor, from_torch_module

    layer = st.one_of(
        st.tuples(st.just("conv"), st.integers(1, 5), st.sampled_from([1, 3]), st.integers(1, 2), st.integers(0, 1), st.booleans()),
        st.tuples(st.just("bn")), st.tuples(st.just("relu")),
        st.tuples(st.just("maxpool"), st.sampled_from([2, 3]), st.integers(1, 2)),
        st.tuples(st.just("avgpool"), st.just(2), st.integers(1, 2)))

    @settings(max_examples=25, deadline=None, suppress_health_check=[HealthCheck.too_slow])
    @given(layers=st.lists(layer, min_size=1, max_size=5), cin=st.integers(1, 3), classes=st.integers(2, 5),
           seed=st.integers(0, 10 ** 6))
    def check(layers, cin, classes, seed):
        torch.manual_seed(seed)
        mods, c, size = [], cin, 10
        for spec in layers:
            kind = spec[0]
            if kind == "conv":
                _, co, k, s, p, bias = spec
                if size + 2 * p < k:
                    continue
                mods.append(torch.nn.Conv2d(c, co, k, s, p, bias=bias))
                c, size = co, (size + 2 * p - k) // s + 1
            elif kind == "bn":
                mods.append(torch.nn.BatchNorm2d(c))
            elif kind == "relu":
                mods.append(torch.nn.ReLU())
            else:
                _, k, s = spec
                if size < k:
                    continue
                mods.append((torch.nn.MaxPool2d if kind == "maxpool" else torch.nn.AvgPool2d)(k, s))
                size = (size - k) // s + 1
        mods += [torch.nn.Flatten(), torch.nn.Linear(c * size * size, classes)]
        g = from_torch_module(torch.nn.Sequential(*mods))
        g.add_loss("SoftmaxCrossEntropy", g.outputs[0])
        x = torch.randn(4, cin, 10, 10)
        y = torch.randint(0, classes, (4,))
        net = GraphNetwork(g).train()
        outs = net(x, label=y)
        outs[-1].backward()
        ref = ReferenceGraphExecutor(g, use_cpp=use_cpp)
        r_outs = ref.inference_and_backprop({g.inputs[0]: x.numpy(), "label": y.numpy()})
        assert np.allclose(r_outs[0], outs[0].detach().numpy(), rtol=1e-3, atol=1e-3), layers
        assert abs(float(r_outs[-1]) - float(outs[-1].detach())) < 1e-3
        for name in g.get_params():
            p = net.tensor(name)
            if p.grad is None or name not in ref.gradients:
                continue
            a, b = ref.gradients[name], p.grad.numpy()
            assert np.allclose(a, b, rtol=2e-2, atol=2e-3 * max(1.0, float(np.abs(b).max()))), (name, layers)

    check()


@pytest.mark.parametrize("batch_first,layers", [(False, 1), (True, 2)])
def test_torch_lstm_models_become_onnx_lstm_nodes(batch_first, layers, tmp_path):
    """A sequence classifier around torch.nn.LSTM (outputs of the last step into a dense layer) traced into ONNX LSTM
    nodes, run by the executor on this package's LSTM layer, and once more from an .onnx file."""
    from eagersgd_b200.graph import GraphNetwork, export_network, from_torch_module, load_onnx

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.lstm = torch.nn.LSTM(6, 8, num_layers=layers, batch_first=batch_first)
            self.fc = torch.nn.Linear(8, 3)

        def forward(self, x):
            out = self.lstm(x)[0]
            last = out.transpose(0, 1)[-1] if batch_first else out[-1]
            return self.fc(last)

    torch.manual_seed(0)
    m = Net().eval()
    x = torch.randn(4, 5, 6) if batch_first else torch.randn(5, 4, 6)
    g = from_torch_module(m, example_inputs=(x,))
    assert [o.op_type for o in g.ops].count("LSTM") == layers
    with torch.no_grad():
        want = m(x)
        got = GraphNetwork(g).eval()(x)
        path = export_network(m, str(tmp_path / "lstm.onnx"), example_inputs=(x,))
        again = GraphNetwork(load_onnx(path)).eval()(x)
    assert torch.allclose(got, want, atol=1e-5) and torch.allclose(again, want, atol=1e-5)


def test_onnx_backend_test_layout_is_read_and_run(tmp_path):
    """Cases in the layout of the ONNX backend test suite (model.onnx, test_data_set_k/{input,output}_i.pb or .npy, in
    folders per kind) are found, read without the onnx package and run on both executors
    (deep500/utils/onnx_interop/onnx_test_parser.py)."""
    from eagersgd_b200.graph import (EmptyVisitor, Graph, OnnxTestData, OnnxTestParser, OpCounter, load_tensor_pb,
                                     save_tensor_pb, write_case)
    rng = np.random.RandomState(0)
    a, b = rng.randn(3, 4).astype(np.float32), rng.randn(3, 4).astype(np.float32)
    g = Graph("test_add")
    g.add("Add", [g.add_input("x"), g.add_input("y")], ["z"])
    g.add_output("z")
    write_case(str(tmp_path / "node"), "add", g, [OnnxTestData([a, b], [a + b]), OnnxTestData([b, b], [2 * b])])
    g2 = Graph("test_gemm")
    g2.add_initializer("w", rng.randn(4, 5).astype(np.float32))
    g2.add("MatMul", [g2.add_input("x"), "w"], ["h"])
    g2.add("Relu", ["h"], ["y"])
    g2.add_output("y")
    write_case(str(tmp_path / "simple"), "test_gemm_relu", g2, [OnnxTestData([a], [np.maximum(a @ g2.initializers["w"], 0)])],
               as_numpy=True)
    p = OnnxTestParser(str(tmp_path))
    assert p.all_tests() == {"node": ["test_add"], "simple": ["test_gemm_relu"]}
    t = p.get_test("add")
    assert len(t.data_sets) == 2 and [op.op_type for op in t.model.ops] == ["Add"]
    assert np.array_equal(t.data_sets[1].inputs[0], b) and np.array_equal(t.data_sets[0].outputs[0], a + b)
    for ex in ("native", "reference"):
        errs = p.run_test("test_add", ex)
        assert len(errs) == 2 and max(max(e) for e in errs) < 1e-6
        assert p.run_test("test_gemm_relu", ex)[0][0] < 1e-4
    with pytest.raises(KeyError, match="there are 2"):
        p.get_test("nothing")
    # tensor files: every element type the reader knows survives, names and scalars included
    for arr in (np.arange(6, dtype=np.int64).reshape(2, 3), np.float64(2.5), np.array([True, False]), a.astype(np.float16)):
        save_tensor_pb(str(tmp_path / "t.pb"), arr, "t")
        back = load_tensor_pb(str(tmp_path / "t.pb"))
        assert back.dtype == np.asarray(arr).dtype and back.shape == np.asarray(arr).shape and np.array_equal(back, arr)
    # a visitor that passes over what it has no method for

    class OnlyRelu(EmptyVisitor):
        def begin(self, graph):
            self.seen = []

        def visit_relu(self, op, graph):
            self.seen.append(op.outputs[0])

        def end(self, graph):
            return self.seen
    assert g2.accept(OnlyRelu()) == ["y"] and g2.accept(OpCounter()) == {"MatMul": 1, "Relu": 1}
