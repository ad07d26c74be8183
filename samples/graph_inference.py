"""Export a network to a model graph, save / load it, visit it and run it.

    python samples/graph_inference.py

Counterpart of the reference's network_inference / onnx parsing samples (deep500 samples/
network_inference.py, utils/onnx_interop/onnx_test_parser.py) on this framework's graph model.
"""
import os
import sys
import tempfile

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from eagersgd_b200.graph import Graph, GraphNetwork, OpCounter, from_torch_resnet  # noqa: E402
from eagersgd_b200.models.resnet import cifar_resnet  # noqa: E402


def main():
    torch.manual_seed(0)
    model = cifar_resnet(20).eval()
    graph = from_torch_resnet(model)
    print("operations:", graph.accept(OpCounter()))
    print("parameters:", sum(v.size for k, v in graph.initializers.items() if k in graph.get_params()))
    with tempfile.TemporaryDirectory() as tmp:
        graph.save(os.path.join(tmp, "resnet20"))
        loaded = Graph.load(os.path.join(tmp, "resnet20"))
    net = GraphNetwork(loaded).eval()
    x = torch.randn(4, 3, 32, 32)
    with torch.no_grad():
        diff = (net(x) - model(x)).abs().max().item()
    print("graph executor vs module: max |difference| = %.2e" % diff)
    assert diff < 1e-3
    loaded.add_loss("SoftmaxCrossEntropy", "logits")
    logits, loss = GraphNetwork(loaded).eval()(x, label=torch.randint(0, 10, (4,)))
    print("with a loss node appended: loss = %.4f" % float(loss.detach()))


if __name__ == "__main__":
    main()
