import numpy as np
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
