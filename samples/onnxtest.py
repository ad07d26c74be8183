"""Run single-operator test cases in the ONNX conformance-test form: a model file plus input / expected-output
tensors, executed on the native executor and on the CPU oracles, compared with an L2 error metric.

    python samples/onnxtest.py [TESTNAME]

The reference picks a case from the onnx package's backend test data (deep500 samples/onnxtest.py:10-34,
utils/onnx_interop/onnx_test_parser.py); that package is not available here, so the cases are generated in the
same shape: ``<case>/model.onnx`` and ``<case>/test_data_set_0/{input_k,output_k}.npy``.
"""
import random
import tempfile
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import numpy as np  # noqa: E402
import torch  # noqa: E402

from eagersgd_b200.graph import Graph, GraphNetwork, ReferenceGraphExecutor, load_onnx, save_onnx  # noqa: E402
from eagersgd_b200.train.metrics import L2Error  # noqa: E402


def _case(root, name, op_type, inputs, attrs, fn):
    g = Graph("test_" + name)
    names = []
    for k, a in enumerate(inputs):
        names.append(g.add_input("in%d" % k))
    g.add(op_type, names, ["out"], **attrs)
    g.add_output("out")
    d = os.path.join(root, "test_" + name, "test_data_set_0")
    os.makedirs(d, exist_ok=True)
    save_onnx(g, os.path.join(root, "test_" + name, "model.onnx"))
    for k, a in enumerate(inputs):
        np.save(os.path.join(d, "input_%d.npy" % k), a)
    np.save(os.path.join(d, "output_0.npy"), fn(*[torch.as_tensor(a) for a in inputs]).numpy())


def generate(root):
    import torch.nn.functional as F
    r = np.random.RandomState(0)
    x = r.randn(2, 3, 8, 8).astype(np.float32)
    _case(root, "relu", "Relu", [x], {}, F.relu)
    _case(root, "add", "Add", [x, x[::-1].copy()], {}, lambda a, b: a + b)
    _case(root, "conv", "Conv", [x, r.randn(4, 3, 3, 3).astype(np.float32)],
          dict(kernel_shape=[3, 3], pads=[1, 1, 1, 1], strides=[1, 1]), lambda a, w: F.conv2d(a, w, padding=1))
    _case(root, "maxpool", "MaxPool", [x], dict(kernel_shape=[2, 2], strides=[2, 2]), lambda a: F.max_pool2d(a, 2, 2))
    _case(root, "averagepool", "AveragePool", [x], dict(kernel_shape=[2, 2], strides=[2, 2]), lambda a: F.avg_pool2d(a, 2, 2))
    _case(root, "matmul", "MatMul", [r.randn(5, 7).astype(np.float32), r.randn(7, 3).astype(np.float32)], {}, torch.matmul)
    _case(root, "softmax", "Softmax", [r.randn(4, 9).astype(np.float32)], dict(axis=1), lambda a: F.softmax(a, 1))
    return sorted(os.listdir(root))


def run_case(root, name):
    case = os.path.join(root, name)
    g = load_onnx(os.path.join(case, "model.onnx"))
    d = os.path.join(case, "test_data_set_0")
    ins = [np.load(os.path.join(d, "input_%d.npy" % k)) for k in range(len(g.inputs))]
    want = np.load(os.path.join(d, "output_0.npy"))
    feeds = dict(zip(g.inputs, ins))
    with torch.no_grad():
        native = GraphNetwork(g).eval()(torch.as_tensor(ins[0]), **{k: torch.as_tensor(v) for k, v in list(feeds.items())[1:]})
    native = (native[0] if isinstance(native, (list, tuple)) else native).numpy()
    oracle = ReferenceGraphExecutor(g, training=False).inference(feeds)[0]
    m = L2Error()
    e_native, e_oracle = m.measure(ins, native, want), m.measure(ins, np.asarray(oracle, np.float32).reshape(want.shape), want)
    print("%-18s L2 error: native %.2e, CPU oracle %.2e" % (name, e_native, e_oracle))
    return e_native, e_oracle


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    root = tempfile.mkdtemp()
    cases = generate(root)
    if argv and argv[0] == "all":
        chosen = cases
    else:
        chosen = [argv[0] if argv and argv[0].startswith("test_") else "test_" + argv[0]] if argv else [random.choice(cases)]
    errs = [run_case(root, c) for c in chosen]
    assert all(max(e) < 1e-3 for e in errs), errs
    return errs


if __name__ == "__main__":
    main()
