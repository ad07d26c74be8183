"""Load a network from an .onnx file and time its inference on an executor.

    python samples/network_inference.py [ONNX FILE] [native|reference]

``native`` runs the graph on this framework's operators (GPU kernels when a GPU is there), ``reference`` on
the CPU oracles.  Without a file, a small ResNet is exported first.  Counterpart of
deep500 samples/network_inference.py:9-28.
"""
import tempfile
import time
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import numpy as np  # noqa: E402
import torch  # noqa: E402

from eagersgd_b200.graph import GraphNetwork, ReferenceGraphExecutor, from_torch_resnet, load_onnx, save_onnx  # noqa: E402
from eagersgd_b200.models.resnet import cifar_resnet  # noqa: E402
from eagersgd_b200.train.metrics import WallclockTime  # noqa: E402


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0].endswith(".onnx"):
        path = argv.pop(0)
    else:
        path = os.path.join(tempfile.mkdtemp(), "resnet8.onnx")
        save_onnx(from_torch_resnet(cifar_resnet(8, 1, 10).eval()), path)
    backend = argv[0] if argv else "native"
    g = load_onnx(path)
    shape = (g.meta.get("shapes", {}).get(g.inputs[0]) or [2, 3, 32, 32])
    shape = [d if isinstance(d, int) and d > 0 else 2 for d in shape] if len(shape) == 4 else [2, 3, 32, 32]
    x = np.random.RandomState(0).randn(*shape).astype(np.float32)
    if backend == "reference":
        ex = ReferenceGraphExecutor(g, training=False)
        run, reruns = (lambda: ex.inference({g.inputs[0]: x})), 3     # the oracles are slow: few reruns
    else:
        net = GraphNetwork(g).eval()
        xt = torch.as_tensor(x)
        run, reruns = (lambda: net(xt)), 20
    with torch.no_grad():
        m = WallclockTime(reruns=reruns, avg_over=1, device=xt.device if backend != "reference" else None)
        ms = m.time_callable(run, warmup=1)
    print("%s on %s (%d nodes): median %.3f ms over %d runs" % (os.path.basename(path), backend, len(g.ops), ms, reruns))
    return ms


if __name__ == "__main__":
    main()
