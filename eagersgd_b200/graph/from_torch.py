"""Any traceable ``torch.nn.Module`` as a model graph (and from there as an ``.onnx`` file).

``torch.fx`` records the module's forward pass symbolically; every recorded call is mapped to the ONNX operator that
the executor and the file writer know.  This stands where the reference exports its PyTorch networks with
``torch.onnx.export`` (deep500/networks/__init__.py:6-21, pytorch_mnist.py, pytorch_deep_mnist.py,
pytorch_wide_resnet.py: ``export_network(name, batch_size, file_path=...)``) — the ``onnx`` package that exporter needs
is not assumed here.  Covered: convolutions, dense layers, batch norm, ReLU / sigmoid / tanh / leaky ReLU, max / average
/ adaptive-average pooling to 1x1, flatten / view(batch, -1), permute / transpose, dropout, softmax / log-softmax,
add / sub / mul / concatenation, stacks of unidirectional LSTM layers (as ONNX LSTM nodes, which the executor runs on
this package's LSTM layer), written as modules or as ``torch.nn.functional`` calls.  Anything else raises with the
node's name.
The ResNets of this package have their own builder (``from_torch_resnet``): their blocks fuse operations in ways a
tracer cannot see through.
"""
from __future__ import annotations

import operator
from typing import Dict, List, Optional

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F

from .ir import Graph


def _pair(v) -> List[int]:
    return [int(v), int(v)] if isinstance(v, int) else [int(a) for a in v]


def _pads(p) -> List[int]:
    a, b = _pair(p)
    return [a, b, a, b]


class _Builder:
    def __init__(self, module: nn.Module, name: str, example_inputs=None):
        import torch.fx as fx
        self.module = module
        self.traced = fx.symbolic_trace(module)
        if example_inputs is not None:            # shapes of every intermediate value: needed where an operator's
            from torch.fx.passes.shape_prop import ShapeProp     # ONNX form depends on the rank (transpose)
            ShapeProp(self.traced).propagate(*example_inputs)
        self.g = Graph(name)
        self.names: Dict[str, str] = {}           # fx node name -> graph tensor name
        self.k = 0

    def fresh(self, stem: str) -> str:
        self.k += 1
        return "%s_%d" % (stem, self.k)

    def init(self, name: str, t: torch.Tensor) -> str:
        return self.g.add_initializer(name, t.detach().float().cpu().numpy())

    def src(self, node) -> str:
        return self.names[node.name]

    def emit(self, node, op_type: str, inputs: List[str], **attrs) -> None:
        out = self.fresh(op_type.lower())
        self.g.add(op_type, inputs, [out], **attrs)
        self.names[node.name] = out

    # ---- modules ---------------------------------------------------------------------------------------------------
    def module_node(self, node, m: nn.Module, x: str) -> None:
        q = node.target.replace(".", "_")
        if isinstance(m, nn.Conv2d):
            if m.groups != 1 or _pair(m.dilation) != [1, 1]:
                raise NotImplementedError("grouped or dilated convolution at %s" % node.target)
            ins = [x, self.init(q + ".weight", m.weight)] + ([self.init(q + ".bias", m.bias)] if m.bias is not None else [])
            self.emit(node, "Conv", ins, kernel_shape=_pair(m.kernel_size), strides=_pair(m.stride), pads=_pads(m.padding))
        elif isinstance(m, nn.Linear):
            bias = m.bias if m.bias is not None else torch.zeros(m.out_features)
            self.emit(node, "Gemm", [x, self.init(q + ".weight", m.weight), self.init(q + ".bias", bias)], transB=1)
        elif isinstance(m, nn.BatchNorm2d):
            w = m.weight if m.weight is not None else torch.ones(m.num_features)
            b = m.bias if m.bias is not None else torch.zeros(m.num_features)
            self.emit(node, "BatchNormalization",
                      [x, self.init(q + ".weight", w), self.init(q + ".bias", b), self.init(q + ".running_mean", m.running_mean),
                       self.init(q + ".running_var", m.running_var)], epsilon=float(m.eps),
                      momentum=1.0 - float(m.momentum if m.momentum is not None else 0.1))
        elif isinstance(m, nn.ReLU):
            self.emit(node, "Relu", [x])
        elif isinstance(m, nn.LeakyReLU):
            self.emit(node, "LeakyRelu", [x], alpha=float(m.negative_slope))
        elif isinstance(m, nn.Sigmoid):
            self.emit(node, "Sigmoid", [x])
        elif isinstance(m, nn.Tanh):
            self.emit(node, "Tanh", [x])
        elif isinstance(m, nn.MaxPool2d):
            self.pool(node, "MaxPool", x, m.kernel_size, m.stride, m.padding)
        elif isinstance(m, nn.AvgPool2d):
            self.pool(node, "AveragePool", x, m.kernel_size, m.stride, m.padding)
        elif isinstance(m, nn.AdaptiveAvgPool2d):
            self.adaptive(node, x, m.output_size)
        elif isinstance(m, nn.Flatten):
            self.emit(node, "Flatten", [x], axis=int(m.start_dim))
        elif isinstance(m, nn.Dropout):
            self.emit(node, "Dropout", [x], ratio=float(m.p))
        elif isinstance(m, nn.Identity):
            self.names[node.name] = x
        elif isinstance(m, nn.Softmax):
            self.emit(node, "Softmax", [x], axis=int(m.dim if m.dim is not None else -1))
        elif isinstance(m, nn.LogSoftmax):
            self.emit(node, "LogSoftmax", [x], axis=int(m.dim if m.dim is not None else -1))
        elif isinstance(m, nn.LSTM):
            self.lstm(node, m, x, q)
        else:
            raise NotImplementedError("no graph operator for module %s (%s)" % (node.target, type(m).__name__))

    def lstm(self, node, m: nn.LSTM, x: str, q: str) -> None:
        """A stack of unidirectional LSTM layers as ONNX LSTM nodes (gates re-ordered from i, f, g, o to ONNX's
        i, o, f, c; the two bias vectors side by side).  The node's value is the pair (outputs, final hidden state
        of the top layer); ``lstm(x)[0]`` picks the outputs."""
        if m.bidirectional or getattr(m, "proj_size", 0) or m.dropout:
            raise NotImplementedError("bidirectional, projected or dropout LSTM at %s" % node.target)
        h = m.hidden_size
        order = torch.cat([torch.arange(0, h), torch.arange(3 * h, 4 * h), torch.arange(h, 2 * h), torch.arange(2 * h, 3 * h)])
        cur = x
        if m.batch_first:
            cur = self.fresh("transpose")
            self.g.add("Transpose", [x], [cur], perm=[1, 0, 2])
        y_h = None
        for l in range(m.num_layers):
            w = getattr(m, "weight_ih_l%d" % l).detach()[order].unsqueeze(0)
            r = getattr(m, "weight_hh_l%d" % l).detach()[order].unsqueeze(0)
            ins = [cur, self.init("%s.W%d" % (q, l), w), self.init("%s.R%d" % (q, l), r)]
            if m.bias:
                b = torch.cat([getattr(m, "bias_ih_l%d" % l).detach()[order], getattr(m, "bias_hh_l%d" % l).detach()[order]])
                ins.append(self.init("%s.B%d" % (q, l), b.unsqueeze(0)))
            y4, y_h = self.fresh("lstm_y"), self.fresh("lstm_h")
            self.g.add("LSTM", ins, [y4, y_h], hidden_size=int(h))
            cur = self.fresh("squeeze")
            self.g.add("Squeeze", [y4], [cur], axes=[1])           # [T, 1, B, H] -> [T, B, H]
        if m.batch_first:
            out = self.fresh("transpose")
            self.g.add("Transpose", [cur], [out], perm=[1, 0, 2])
            cur = out
        self.names[node.name] = (cur, y_h)

    def pool(self, node, op_type, x, k, s, p) -> None:
        self.emit(node, op_type, [x], kernel_shape=_pair(k), strides=_pair(s if s is not None else k), pads=_pads(p))

    def adaptive(self, node, x, size) -> None:
        if _pair(size) != [1, 1]:
            raise NotImplementedError("adaptive pooling to %s at %s (only 1x1 has an ONNX operator)" % (size, node.name))
        self.emit(node, "GlobalAveragePool", [x])

    # ---- functions and methods ---------------------------------------------------------------------------------------
    def function_node(self, node) -> None:
        t, a, kw = node.target, node.args, node.kwargs
        arg = lambda i, key, default=None: a[i] if len(a) > i else kw.get(key, default)
        x = self.src(a[0]) if a and hasattr(a[0], "name") and isinstance(self.names.get(a[0].name), str) else None
        if t in (F.relu, torch.relu):
            self.emit(node, "Relu", [x])
        elif t in (torch.sigmoid, F.sigmoid):
            self.emit(node, "Sigmoid", [x])
        elif t in (torch.tanh, F.tanh):
            self.emit(node, "Tanh", [x])
        elif t is F.leaky_relu:
            self.emit(node, "LeakyRelu", [x], alpha=float(arg(1, "negative_slope", 0.01)))
        elif t is F.max_pool2d:
            self.pool(node, "MaxPool", x, arg(1, "kernel_size"), arg(2, "stride"), arg(3, "padding", 0))
        elif t is F.avg_pool2d:
            self.pool(node, "AveragePool", x, arg(1, "kernel_size"), arg(2, "stride"), arg(3, "padding", 0))
        elif t is F.adaptive_avg_pool2d:
            self.adaptive(node, x, arg(1, "output_size"))
        elif t is torch.flatten:
            self.emit(node, "Flatten", [x], axis=int(arg(1, "start_dim", 0)))
        elif t is F.dropout:
            self.emit(node, "Dropout", [x], ratio=float(arg(1, "p", 0.5)))
        elif t is F.softmax:
            self.emit(node, "Softmax", [x], axis=int(arg(1, "dim", -1)))
        elif t is F.log_softmax:
            self.emit(node, "LogSoftmax", [x], axis=int(arg(1, "dim", -1)))
        elif t in (operator.add, torch.add, operator.sub, torch.sub, operator.mul, torch.mul):
            kind = {operator.add: "Add", torch.add: "Add", operator.sub: "Sub", torch.sub: "Sub"}.get(t, "Mul")
            self.emit(node, kind, [self.operand(v) for v in a[:2]])
        elif t is torch.cat:
            self.emit(node, "Concat", [self.src(v) for v in a[0]], axis=int(arg(1, "dim", 0)))
        elif t is operator.getitem and isinstance(self.names.get(a[0].name), tuple):
            picked = self.names[a[0].name][a[1]] if isinstance(a[1], int) else None
            if picked is None:
                raise NotImplementedError("only lstm(x)[0] and lstm(x)[1] are known at %s" % node.name)
            self.names[node.name] = picked if isinstance(picked, str) else (picked,)
        elif t is operator.getitem and isinstance(a[1], int) and a[1] < 0 and x is not None:
            # x[-1] on the leading axis (the last time step of [T, B, H])
            idx = self.fresh("const")
            self.g.add("Constant", [], [idx], value=np.asarray(a[1], dtype=np.int64))
            self.emit(node, "Gather", [x, idx], axis=0)
        else:
            raise NotImplementedError("no graph operator for the call %s at %s" % (getattr(t, "__name__", t), node.name))

    def operand(self, v) -> str:
        if hasattr(v, "name"):
            return self.src(v)
        out = self.fresh("const")                              # a python number next to a tensor
        self.g.add("Constant", [], [out], value=np.asarray(v, dtype=np.float32))
        return out

    def method_node(self, node) -> None:
        x = self.src(node.args[0])
        if node.target == "flatten":
            self.emit(node, "Flatten", [x], axis=int(node.args[1] if len(node.args) > 1 else node.kwargs.get("start_dim", 0)))
        elif node.target in ("view", "reshape") and len(node.args) == 3 and node.args[2] == -1:
            self.emit(node, "Flatten", [x], axis=1)            # x.view(batch, -1)
        elif node.target in ("relu", "sigmoid", "tanh"):
            self.emit(node, node.target.capitalize(), [x])
        elif node.target in ("contiguous", "float", "detach"):
            self.names[node.name] = x
        elif node.target == "permute":
            dims = node.args[1] if isinstance(node.args[1], (tuple, list)) else node.args[1:]
            self.emit(node, "Transpose", [x], perm=[int(d) for d in dims])
        elif node.target == "transpose":
            meta = node.args[0].meta.get("tensor_meta") if hasattr(node.args[0], "meta") else None
            if meta is None:
                raise NotImplementedError("x.transpose() at %s needs the rank of x: pass example_inputs" % node.name)
            perm = list(range(len(meta.shape)))
            d0, d1 = int(node.args[1]) % len(perm), int(node.args[2]) % len(perm)
            perm[d0], perm[d1] = perm[d1], perm[d0]
            self.emit(node, "Transpose", [x], perm=perm)
        else:
            raise NotImplementedError("no graph operator for the method .%s() at %s" % (node.target, node.name))

    def build(self) -> Graph:
        mods = dict(self.traced.named_modules())
        for node in self.traced.graph.nodes:
            if node.op == "placeholder":
                self.names[node.name] = self.g.add_input(node.name)
            elif node.op == "call_module":
                self.module_node(node, mods[node.target], self.src(node.args[0]))
            elif node.op == "call_function":
                self.function_node(node)
            elif node.op == "call_method":
                self.method_node(node)
            elif node.op == "get_attr":
                obj = self.traced
                for part in node.target.split("."):
                    obj = getattr(obj, part)
                self.names[node.name] = self.init(node.target.replace(".", "_"), obj)
            elif node.op == "output":
                outs = node.args[0] if isinstance(node.args[0], (tuple, list)) else [node.args[0]]
                for o in outs:
                    self.g.add_output(self.src(o))
        return self.g


def from_torch_module(module: nn.Module, name: Optional[str] = None, example_inputs=None) -> Graph:
    """The forward pass of ``module`` as a graph whose initializers are the module's current weights.
    ``example_inputs`` (a tuple of tensors) lets the tracer know every intermediate shape; a few operators need it."""
    return _Builder(module, name or type(module).__name__, example_inputs).build()


def export_network(name_or_module, file_path=None, example_inputs=None, **kwargs) -> str:
    """Write a network as an ``.onnx`` file and return the path: ``name_or_module`` is a module or a name that
    ``models.create_model`` knows ("simple_cnn", "simple_mnist", "deep_mnist", "wide_resnet", "resnet"); keyword
    arguments go to the constructor.  In the reference's call form the second argument is a batch size and the file
    goes to ``file_path=`` or, by default, ``<name>.onnx`` in the working directory
    (``export_network(name, batch_size, classes=..., shape=...)``, deep500/networks/__init__.py:6-21)."""
    from .onnx_io import save_onnx
    if file_path is None or isinstance(file_path, int):
        file_path = kwargs.pop("file_path", None) or "%s.onnx" % (name_or_module if isinstance(name_or_module, str) else
                                                                 type(name_or_module).__name__.lower())
    if isinstance(name_or_module, nn.Module):
        module = name_or_module
    else:
        from ..models import create_model
        shape = kwargs.get("shape")
        module = create_model(name_or_module, **kwargs)
        if example_inputs is None and shape is not None:
            example_inputs = (torch.zeros(1, *shape),)
    module = module.eval()
    from ..models.resnet import ResNet
    if isinstance(module, ResNet):
        from .executor import from_torch_resnet
        g = from_torch_resnet(module)
    else:
        g = from_torch_module(module, example_inputs=example_inputs)
    save_onnx(g, file_path)
    return file_path
