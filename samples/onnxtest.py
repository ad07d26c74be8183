"""Run single-operator test cases in the ONNX conformance-test form: a model file plus input / expected-output
tensors, executed on the native executor and on the CPU oracles, compared with an L2 error metric.

    python samples/onnxtest.py [TESTNAME]

The reference picks a case from the onnx package's backend test data (deep500 samples/onnxtest.py:10-34,
utils/onnx_interop/onnx_test_parser.py); that package is not available here, so the cases are generated in the
same layout — ``<case>/model.onnx`` and ``<case>/test_data_set_0/{input_k,output_k}.pb`` (serialized tensors) — and read
back through ``eagersgd_b200.graph.OnnxTestParser``, which reads a copy of the real suite's data just as well.
"""
import random
import tempfile
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import numpy as np  # noqa: E402
import torch  # noqa: E402

from eagersgd_b200.graph import Graph, OnnxTestData, OnnxTestParser, write_case  # noqa: E402


def _case(root, name, op_type, inputs, attrs, fn):
    g = Graph("test_" + name)
    names = [g.add_input("in%d" % k) for k in range(len(inputs))]
    g.add(op_type, names, ["out"], **attrs)
    g.add_output("out")
    want = fn(*[torch.as_tensor(a) for a in inputs]).numpy()
    write_case(root, name, g, [OnnxTestData(list(inputs), [want])])      # model.onnx + test_data_set_0/{input,output}_k.pb


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
    parser = OnnxTestParser(root)
    e_native = parser.run_test(name, "native")[0][0]
    e_oracle = parser.run_test(name, "reference")[0][0]
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
