"""Operator and model test cases in the layout of the ONNX backend test suite.

A case is a directory ``test_<name>/`` with ``model.onnx`` and one or more ``test_data_set_<k>/`` folders that hold
``input_<i>.pb`` / ``output_<i>.pb`` — each a serialized ``TensorProto`` — or, for the cases that suite keeps as
arrays, ``input_<i>.npy`` / ``output_<i>.npy`` (``.npz`` archives ``inputs.npz`` / ``outputs.npz`` are read too).
``OnnxTestParser`` finds the cases under a root directory, reads them without the ``onnx`` package (the wire-format
reader of ``onnx_io`` does the decoding) and runs them on the native executor or on the CPU oracles.

The reference's counterpart walks the test data that ships inside the ``onnx`` package
(deep500/utils/onnx_interop/onnx_test_parser.py:15-97: ``get_test``, ``all_tests``, numpy and protobuf data sets);
here the root directory is an argument, so a copy of that data, or cases written with ``write_case``, can be used.
"""
from __future__ import annotations

import glob
import os
import re
from collections import namedtuple
from typing import Callable, Dict, List, Optional, Sequence

import numpy as np

from .ir import Graph
from .onnx_io import _enc_tensor, _parse_tensor, load_onnx, save_onnx

OnnxTestData = namedtuple("OnnxTestData", ["inputs", "outputs"])
OnnxTest = namedtuple("OnnxTest", ["model", "data_sets"])


def load_tensor_pb(path: str) -> np.ndarray:
    """One ``TensorProto`` file as an array."""
    with open(path, "rb") as f:
        return _parse_tensor(f.read())[1]


def save_tensor_pb(path: str, array, name: str = "") -> None:
    with open(path, "wb") as f:
        f.write(_enc_tensor(name, np.asarray(array)))


def write_case(root: str, name: str, graph: Graph, data_sets: Sequence[OnnxTestData], as_numpy: bool = False) -> str:
    """Write ``test_<name>`` under ``root`` in the suite's layout and return its directory."""
    case = os.path.join(root, name if name.startswith("test_") else "test_" + name)
    os.makedirs(case, exist_ok=True)
    save_onnx(graph, os.path.join(case, "model.onnx"))
    for k, ds in enumerate(data_sets):
        d = os.path.join(case, "test_data_set_%d" % k)
        os.makedirs(d, exist_ok=True)
        for kind, arrays, names in (("input", ds.inputs, graph.inputs), ("output", ds.outputs, graph.outputs)):
            for i, a in enumerate(arrays):
                if as_numpy:
                    np.save(os.path.join(d, "%s_%d.npy" % (kind, i)), np.asarray(a))
                else:
                    save_tensor_pb(os.path.join(d, "%s_%d.pb" % (kind, i)), a, names[i] if i < len(names) else "")
    return case


def _numbered(directory: str, kind: str) -> List[np.ndarray]:
    found = {}
    for path in glob.glob(os.path.join(directory, kind + "_*")):
        m = re.match(r"^%s_(\d+)\.(pb|npy)$" % kind, os.path.basename(path))
        if m:
            found[int(m.group(1))] = load_tensor_pb(path) if m.group(2) == "pb" else np.load(path)
    archive = os.path.join(directory, kind + "s.npz")
    if not found and os.path.exists(archive):
        with np.load(archive) as z:
            return [z[k] for k in z.files]
    return [found[k] for k in sorted(found)]


class OnnxTestParser:
    def __init__(self, root: str):
        self.root = root
        self.tests: Dict[str, str] = {}
        for model in sorted(glob.glob(os.path.join(root, "**", "model.onnx"), recursive=True)):
            case = os.path.dirname(model)
            self.tests[os.path.basename(case)] = case

    def all_tests(self) -> Dict[str, List[str]]:
        """Case names by the folder they were found in (the suite's kinds: node, real, simple, ...)."""
        out: Dict[str, List[str]] = {}
        for name, case in self.tests.items():
            kind = os.path.relpath(os.path.dirname(case), self.root)
            out.setdefault("" if kind == "." else kind, []).append(name)
        return out

    def get_test(self, name: str) -> OnnxTest:
        if name not in self.tests and "test_" + name in self.tests:
            name = "test_" + name
        if name not in self.tests:
            raise KeyError("no test case %r under %s (there are %d)" % (name, self.root, len(self.tests)))
        case = self.tests[name]
        sets = []
        for d in sorted(glob.glob(os.path.join(case, "test_data_set_*")),
                        key=lambda p: int(p.rsplit("_", 1)[1]) if p.rsplit("_", 1)[1].isdigit() else 0):
            sets.append(OnnxTestData(_numbered(d, "input"), _numbered(d, "output")))
        return OnnxTest(load_onnx(os.path.join(case, "model.onnx")), sets)

    def run_test(self, name: str, executor: str = "native", metric: Optional[Callable] = None) -> List[List[float]]:
        """Run every data set of a case; returns, per data set, the error of each output against the expected one
        (L2 distance by default).  ``executor``: "native" (``GraphNetwork``, the framework's own operators) or
        "reference" (the numpy / C++ oracles)."""
        import torch

        from ..train.metrics import L2Error
        from .executor import GraphNetwork
        from .reference_executor import ReferenceGraphExecutor
        test = self.get_test(name)
        g = test.model
        measure = metric or (lambda got, want: L2Error().measure(None, got, want))
        results = []
        for ds in test.data_sets:
            feeds = dict(zip(g.inputs, ds.inputs))
            if executor == "reference":
                outs = ReferenceGraphExecutor(g, training=False).inference(feeds)
            else:
                if not g.initializers:
                    g.add_initializer("_device_anchor", np.zeros(1, np.float32))      # the executor asks a parameter for its device
                net = GraphNetwork(g, trainable_only_used=False).eval()
                first, rest = g.inputs[0], {k: torch.as_tensor(v) for k, v in feeds.items() if k != g.inputs[0]}
                with torch.no_grad():
                    outs = net(torch.as_tensor(feeds[first]), **rest)
                outs = list(outs) if isinstance(outs, (list, tuple)) else [outs]
                outs = [o.detach().cpu().numpy() for o in outs]
            results.append([float(measure(np.asarray(o, dtype=np.asarray(w).dtype).reshape(np.asarray(w).shape), np.asarray(w)))
                            for o, w in zip(outs, ds.outputs)])
        return results
