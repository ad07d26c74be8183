"""Model graphs: an ONNX-shaped object model with visitor dispatch.

``Graph`` holds ``Operation`` nodes (op_type, named inputs / outputs, attributes), initializers
(named weight tensors) and the graph inputs / outputs; ``Visitor`` dispatches ``visit_<op_type>``
per node in topological order.  It is the object model the reference builds from ONNX protobufs
(deep500/utils/onnx_interop/onnx_objects.py, generated_operators.py, onnx_base_visitor.py,
operations_visitor.py, losses.py, extended_operations.py) without the protobuf dependency: graphs
are built programmatically, read from ``.onnx`` files (onnx_io.py) or loaded from a JSON + NPZ pair in the
same schema.  Nodes of standard operators are instances of that operator's class (onnx_ops.py).
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, List, Optional, Sequence

import numpy as np

# op types understood by the executor (ONNX names) plus the reference's extensions
STANDARD_OPS = ("Conv", "BatchNormalization", "Relu", "MaxPool", "AveragePool", "GlobalAveragePool", "Gemm", "MatMul",
                "Add", "Sum", "Flatten", "Reshape", "Squeeze", "Unsqueeze", "Softmax", "Dropout", "Identity", "Concat",
                "Sub", "Mul", "Div", "Neg", "Abs", "Exp", "Log", "Sqrt", "Pow", "Sigmoid", "Tanh", "LeakyRelu", "Transpose",
                "LogSoftmax", "Clip", "ReduceMean", "ReduceSum", "Constant", "Pad", "LRN",
                # comparisons, logic and selection
                "Equal", "Greater", "GreaterOrEqual", "Less", "LessOrEqual", "And", "Or", "Xor", "Not", "Where", "IsNaN",
                "Max", "Min", "Mean",
                # the rest of the unary maths and activations
                "Floor", "Ceil", "Round", "Sign", "Reciprocal", "Erf", "Sin", "Cos", "Softplus", "Softsign", "Elu", "Selu",
                "HardSigmoid", "PRelu", "ThresholdedRelu", "Cast",
                # reductions and selection by value
                "ReduceMax", "ReduceMin", "ReduceProd", "ReduceL1", "ReduceL2", "ReduceSumSquare", "ReduceLogSumExp",
                "ArgMax", "ArgMin", "TopK", "CumSum",
                # shapes and data movement
                "Shape", "Size", "Expand", "Tile", "Gather", "Slice", "Split", "DepthToSpace", "SpaceToDepth",
                "ConstantOfShape", "Range", "OneHot",
                # layers
                "ConvTranspose", "InstanceNormalization", "GlobalMaxPool", "LpNormalization", "Resize", "Upsample",
                "LSTM")
LOSS_OPS = ("SoftmaxCrossEntropy", "CrossEntropy", "MeanSquaredError")
EXTENSION_OPS = ("StopGradient", "AllReduceGradients", "ConsistentParameterServerGradients",
                 "InconsistentParameterServerGradients")


class Operation:
    def __init__(self, op_type: str, inputs: Sequence[str], outputs: Sequence[str], name: Optional[str] = None, **attrs):
        self.op_type, self.inputs, self.outputs = op_type, list(inputs), list(outputs)
        self.name = name or "%s_%s" % (op_type, outputs[0])
        self.attrs: Dict[str, Any] = dict(attrs)

    def accept(self, visitor: "Visitor", graph: "Graph"):
        fn = getattr(visitor, "visit_" + self.op_type.lower(), None)
        return fn(self, graph) if fn is not None else visitor.visit_default(self, graph)

    def to_dict(self) -> dict:
        return {"op_type": self.op_type, "name": self.name, "inputs": self.inputs, "outputs": self.outputs,
                "attrs": self.attrs}

    def __repr__(self):
        return "%s(%s -> %s)" % (self.op_type, ", ".join(self.inputs), ", ".join(self.outputs))


class Graph:
    def __init__(self, name: str = "graph"):
        self.name = name
        self.ops: List[Operation] = []
        self.initializers: Dict[str, np.ndarray] = {}
        self.inputs: List[str] = []
        self.outputs: List[str] = []

    # ---- construction ----------------------------------------------------------
    def add_input(self, name: str) -> str:
        self.inputs.append(name)
        return name

    def add_initializer(self, name: str, value: np.ndarray) -> str:
        self.initializers[name] = np.asarray(value)
        return name

    def add(self, op_type: str, inputs: Sequence[str], outputs: Sequence[str], **attrs) -> Operation:
        from .onnx_ops import make_operation
        op = make_operation(op_type, inputs, outputs, **attrs)     # the operator's own class where ONNX defines it
        self.ops.append(op)
        return op

    def add_output(self, name: str):
        if name not in self.outputs:
            self.outputs.append(name)

    def add_loss(self, kind: str, prediction: str, label: str = "label", loss: str = "loss") -> str:
        """Append a loss operation (losses.py of the reference adds them to a parsed model)."""
        assert kind in LOSS_OPS
        if label not in self.inputs:
            self.add_input(label)
        self.add(kind, [prediction, label], [loss])
        self.add_output(loss)
        return loss

    # ---- queries ---------------------------------------------------------------
    def get_params(self) -> List[str]:
        used = {i for op in self.ops for i in op.inputs}
        return [n for n in self.initializers if n in used]

    def producers(self) -> Dict[str, Operation]:
        return {o: op for op in self.ops for o in op.outputs}

    def topological(self) -> List[Operation]:
        ready = set(self.inputs) | set(self.initializers)
        pending, order = list(self.ops), []
        while pending:
            progressed = False
            for op in list(pending):
                if all((i in ready) or i == "" for i in op.inputs):
                    order.append(op)
                    ready.update(op.outputs)
                    pending.remove(op)
                    progressed = True
            if not progressed:
                raise ValueError("graph has a cycle or an undefined input: %s" % pending[0])
        return order

    def accept(self, visitor: "Visitor"):
        visitor.begin(self)
        for op in self.topological():
            op.accept(visitor, self)
        return visitor.end(self)

    # ---- serialisation ------------------------------------------------------------
    def save(self, path: str):
        base = os.path.splitext(path)[0]
        with open(base + ".json", "w") as f:
            json.dump({"name": self.name, "inputs": self.inputs, "outputs": self.outputs,
                       "ops": [op.to_dict() for op in self.ops], "initializers": sorted(self.initializers)}, f)
        np.savez(base + ".npz", **self.initializers)

    @staticmethod
    def load(path: str) -> "Graph":
        base = os.path.splitext(path)[0]
        d = json.load(open(base + ".json"))
        g = Graph(d["name"])
        g.inputs, g.outputs = d["inputs"], d["outputs"]
        for o in d["ops"]:
            from .onnx_ops import make_operation
            g.ops.append(make_operation(o["op_type"], o["inputs"], o["outputs"], o["name"], **o["attrs"]))
        z = np.load(base + ".npz")
        g.initializers = {k: z[k] for k in z.files}
        return g

    def to_dot(self) -> str:
        lines = ["digraph %s {" % self.name]
        for op in self.ops:
            lines.append('  "%s" [label="%s"];' % (op.name, op.op_type))
            prod = self.producers()
            for i in op.inputs:
                if i in prod:
                    lines.append('  "%s" -> "%s";' % (prod[i].name, op.name))
        return "\n".join(lines + ["}"])


class Visitor:
    """Base visitor: override ``visit_<op_type lower-case>``; unknown ops go to ``visit_default``."""

    def begin(self, graph: Graph): ...

    def end(self, graph: Graph):
        return None

    def visit_default(self, op: Operation, graph: Graph):
        raise NotImplementedError("no visitor method for op type %s" % op.op_type)


class EmptyVisitor(Visitor):
    """A visitor that passes over operators it has no method for instead of raising (the reference's
    ``EmptyOnnxBaseVisitor``, deep500/utils/onnx_interop/onnx_base_visitor.py): override the few you care about."""

    def visit_default(self, op: Operation, graph: Graph):
        return None


class OpCounter(Visitor):
    """Counts operations per type (an 'empty operations visitor' that does something useful)."""

    def begin(self, graph):
        self.counts: Dict[str, int] = {}

    def visit_default(self, op, graph):
        self.counts[op.op_type] = self.counts.get(op.op_type, 0) + 1

    def end(self, graph):
        return self.counts
