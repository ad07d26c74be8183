"""Executing a model graph with this framework's operators.

``GraphNetwork`` turns a ``Graph`` into a ``torch.nn.Module`` whose parameters are the graph's
initializers and whose forward pass visits the operations in topological order, mapping every
ONNX op type to the hand-written kernels (through ``ops.functional``) or a PyTorch op.  Together
with ``train.executor.GraphExecutor`` this is the counterpart of the reference's per-framework
network builders and graph executors (deep500/frameworks/pytorch/pytorch_visitor.py,
pytorch_network.py, pytorch_graph_executor.py; reference/reference_graph_executor.py:34-47) and
of its gradient extension ops (extended_operations.py:27-77), which no backend there implements.
"""
from __future__ import annotations

from typing import Dict

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as ops
from .executor_ops import MoreOperators, _ints
from .ir import Graph, Visitor


class _Forward(MoreOperators, Visitor):
    def __init__(self, net: "GraphNetwork", feeds: Dict[str, torch.Tensor]):
        self.net, self.v = net, dict(feeds)

    def begin(self, graph):
        for name in graph.initializers:
            self.v[name] = self.net.tensor(name)

    def end(self, graph):
        return self.v

    def _in(self, op, k):
        return self.v[op.inputs[k]] if k < len(op.inputs) and op.inputs[k] != "" else None

    def _out(self, op, value):
        self.v[op.outputs[0]] = value

    def visit_conv(self, op, g):
        stride = op.attrs.get("strides", [1, 1])[0]
        pad = op.attrs.get("pads", [0, 0, 0, 0])[0]
        x, w, b = self._in(op, 0), self._in(op, 1), self._in(op, 2)
        if b is None:
            y, _ = ops.conv2d(x, w, stride, pad)
        else:
            y = F.conv2d(x, w, b, stride, pad)
        self._out(op, y)

    def visit_batchnormalization(self, op, g):
        x, gamma, beta, mean, var = (self._in(op, k) for k in range(5))
        self._out(op, ops.bn_act(x, gamma, beta, mean, var, 1.0 - op.attrs.get("momentum", 0.9), relu=False,
                                 training=self.net.training))

    def visit_relu(self, op, g): self._out(op, F.relu(self._in(op, 0)))

    def visit_maxpool(self, op, g):
        k, s = op.attrs.get("kernel_shape", [2, 2])[0], op.attrs.get("strides", [1, 1])[0]
        p = op.attrs.get("pads", [0, 0, 0, 0])[0]
        x = self._in(op, 0)
        self._out(op, ops.max_pool_3x3_s2(x) if (k, s, p) == (3, 2, 1) else F.max_pool2d(x, k, s, p))

    def visit_averagepool(self, op, g):
        k, s = op.attrs.get("kernel_shape", [2, 2])[0], op.attrs.get("strides", [1, 1])[0]
        self._out(op, F.avg_pool2d(self._in(op, 0), k, s, op.attrs.get("pads", [0, 0, 0, 0])[0]))

    def visit_globalaveragepool(self, op, g):
        y = ops.global_avg_pool(self._in(op, 0))
        self._out(op, y.view(y.shape[0], y.shape[1], 1, 1))

    def visit_gemm(self, op, g):
        a, b, c = self._in(op, 0), self._in(op, 1), self._in(op, 2)
        if op.attrs.get("transA", 0):
            a = a.t()
        w = b if op.attrs.get("transB", 0) else b.t()          # ops.linear wants [out, in]
        self._out(op, ops.linear(a, w.contiguous() if not op.attrs.get("transB", 0) else w, c))

    def visit_matmul(self, op, g): self._out(op, self._in(op, 0) @ self._in(op, 1))
    def visit_add(self, op, g): self._out(op, self._in(op, 0) + self._in(op, 1))
    def visit_sum(self, op, g): self._out(op, sum(self.v[i] for i in op.inputs))
    def visit_flatten(self, op, g): self._out(op, torch.flatten(self._in(op, 0), op.attrs.get("axis", 1)))
    def visit_reshape(self, op, g):
        x, shape = self._in(op, 0), (_ints(self._in(op, 1)) if self._in(op, 1) is not None else list(op.attrs["shape"]))
        shape = [x.shape[i] if d == 0 and not op.attrs.get("allowzero", 0) else d for i, d in enumerate(shape)]
        self._out(op, x.reshape(shape))

    def visit_squeeze(self, op, g):
        x, axes = self._in(op, 0), self._axes(op)
        if axes is None:
            return self._out(op, x.squeeze())
        for a in sorted((a % x.dim() for a in axes), reverse=True):
            x = x.squeeze(a)
        self._out(op, x)

    def visit_unsqueeze(self, op, g):
        x, axes = self._in(op, 0), self._axes(op)
        for a in sorted(a % (x.dim() + len(axes)) for a in axes):
            x = x.unsqueeze(a)
        self._out(op, x)
    def visit_softmax(self, op, g): self._out(op, F.softmax(self._in(op, 0).float(), op.attrs.get("axis", -1)))
    def visit_identity(self, op, g): self._out(op, self._in(op, 0))
    def visit_concat(self, op, g): self._out(op, torch.cat([self.v[i] for i in op.inputs], op.attrs.get("axis", 1)))

    # elementwise / shape operators of the reference's PyTorch visitor (pytorch_visitor.py) beyond the ResNet set
    def visit_sub(self, op, g): self._out(op, self._in(op, 0) - self._in(op, 1))
    def visit_mul(self, op, g): self._out(op, self._in(op, 0) * self._in(op, 1))
    def visit_div(self, op, g): self._out(op, self._in(op, 0) / self._in(op, 1))
    def visit_neg(self, op, g): self._out(op, -self._in(op, 0))
    def visit_abs(self, op, g): self._out(op, self._in(op, 0).abs())
    def visit_exp(self, op, g): self._out(op, self._in(op, 0).exp())
    def visit_log(self, op, g): self._out(op, self._in(op, 0).log())
    def visit_sqrt(self, op, g): self._out(op, self._in(op, 0).sqrt())
    def visit_pow(self, op, g): self._out(op, self._in(op, 0) ** self._in(op, 1))
    def visit_sigmoid(self, op, g): self._out(op, torch.sigmoid(self._in(op, 0)))
    def visit_tanh(self, op, g): self._out(op, torch.tanh(self._in(op, 0)))
    def visit_leakyrelu(self, op, g): self._out(op, F.leaky_relu(self._in(op, 0), op.attrs.get("alpha", 0.01)))
    def visit_transpose(self, op, g): self._out(op, self._in(op, 0).permute(*op.attrs["perm"]))
    def visit_logsoftmax(self, op, g): self._out(op, F.log_softmax(self._in(op, 0).float(), op.attrs.get("axis", -1)))

    def visit_clip(self, op, g):
        self._out(op, self._in(op, 0).clamp(op.attrs.get("min", None), op.attrs.get("max", None)))

    def visit_reducemean(self, op, g): self._reduce(op, lambda x, a, k: x.mean(dim=a, keepdim=k))
    def visit_reducesum(self, op, g): self._reduce(op, lambda x, a, k: x.sum(dim=a, keepdim=k))

    def visit_constant(self, op, g):
        value = np.asarray(op.attrs["value"])
        if value.dtype == np.float64:                 # python floats: ONNX constants are float32 unless typed
            value = value.astype(np.float32)
        self._out(op, torch.as_tensor(value).to(next(self.net.parameters()).device))

    def visit_pad(self, op, g):
        pads = op.attrs["pads"]                       # ONNX order: begins of all axes, then ends
        n = len(pads) // 2
        torch_pads = []
        for ax in reversed(range(n)):
            torch_pads += [pads[ax], pads[ax + n]]
        self._out(op, F.pad(self._in(op, 0), torch_pads, value=op.attrs.get("value", 0.0)))

    def visit_lrn(self, op, g):
        self._out(op, F.local_response_norm(self._in(op, 0), op.attrs["size"], op.attrs.get("alpha", 1e-4),
                                            op.attrs.get("beta", 0.75), op.attrs.get("bias", 1.0)))

    def visit_dropout(self, op, g):
        self._out(op, F.dropout(self._in(op, 0), op.attrs.get("ratio", 0.5), self.net.training))

    # losses
    def visit_softmaxcrossentropy(self, op, g):
        logits = self._in(op, 0)
        self._out(op, ops.softmax_cross_entropy(logits if logits.dtype == torch.float32 else logits.float(),
                                                self._in(op, 1)))

    def visit_crossentropy(self, op, g):
        p = self._in(op, 0).float().clamp_min(1e-12)
        self._out(op, F.nll_loss(p.log(), self._in(op, 1)))

    def visit_meansquarederror(self, op, g):
        self._out(op, F.mse_loss(self._in(op, 0).float(), self._in(op, 1).float()))

    # extensions
    def visit_stopgradient(self, op, g): self._out(op, self._in(op, 0).detach())

    def visit_allreducegradients(self, op, g):
        """Identity in the forward pass; the gradient flowing back is averaged over the group."""
        self._out(op, _AllReduceGrad.apply(self._in(op, 0), self.net.group))


    def visit_consistentparameterservergradients(self, op, g):
        """Identity forward; backward the gradients of all ranks meet at rank 0, are averaged there and sent back
        (extended_operations.py:27-77 declares the operation; no backend of the reference implements it)."""
        self._out(op, _ParameterServerGrad.apply(self._in(op, 0), self.net.group))

    def visit_inconsistentparameterservergradients(self, op, g):
        """Identity in both directions: with an inconsistent parameter server every rank applies its own
        gradient and the exchange happens in the optimizer (``optim.distributed.InconsistentParameterServer``)."""
        self._out(op, self._in(op, 0).view_as(self._in(op, 0)))


class _ParameterServerGrad(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        gr = ctx.group
        if gr is not None and gr.world > 1:
            g = g.contiguous()
            gr.sync_all_at_root(g, average=True)
            gr.bcast(g, 0)
        return g, None


class _AllReduceGrad(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        if ctx.group is not None and ctx.group.world > 1:
            g = g.contiguous()
            ctx.group.sync_all(g, average=True)
        return g, None


class GraphNetwork(nn.Module):
    def __init__(self, graph: Graph, group=None, trainable_only_used: bool = True):
        super().__init__()
        self.graph, self.group = graph, group
        self._names: Dict[str, str] = {}
        bn_stats = {op.inputs[k] for op in graph.ops if op.op_type == "BatchNormalization" for k in (3, 4)}
        for i, (name, value) in enumerate(graph.initializers.items()):
            t = torch.as_tensor(np.asarray(value))
            key = "p%d" % i
            self._names[name] = key
            if name in bn_stats or not t.is_floating_point():
                self.register_buffer(key, t.clone())
            else:
                self.register_parameter(key, nn.Parameter(t.clone()))

    def tensor(self, name: str) -> torch.Tensor:
        return getattr(self, self._names[name])

    def forward(self, x, **feeds):
        values = {self.graph.inputs[0]: x}
        values.update(feeds)
        out = self.graph.accept(_Forward(self, values))
        res = [out[o] for o in self.graph.outputs if o in out]
        return res[0] if len(res) == 1 else tuple(res)

    def export_initializers(self) -> Dict[str, np.ndarray]:
        return {n: self.tensor(n).detach().float().cpu().numpy() for n in self.graph.initializers}


def from_torch_resnet(model) -> Graph:
    """Graph of a ``models.resnet.ResNet`` (v1): the creation-order registry gives the node order."""
    g = Graph("resnet")
    x = g.add_input("input")
    cnt = {"conv": 0, "bn": 0}

    def conv(mod, inp):
        k = cnt["conv"]
        cnt["conv"] += 1
        w = g.add_initializer("conv%d.weight" % k, mod.weight.detach().float().numpy())
        out = "conv%d.out" % k
        g.add("Conv", [inp, w], [out], strides=[mod.stride[0]] * 2, pads=[mod.padding[0]] * 4,
              kernel_shape=list(mod.kernel_size))
        return out

    def bn(mod, inp):
        k = cnt["bn"]
        cnt["bn"] += 1
        names = [g.add_initializer("bn%d.%s" % (k, n), t.detach().float().numpy())
                 for n, t in (("gamma", mod.weight), ("beta", mod.bias), ("mean", mod.running_mean),
                              ("var", mod.running_var))]
        out = "bn%d.out" % k
        g.add("BatchNormalization", [inp] + names, [out], momentum=1.0 - mod.momentum, epsilon=mod.eps)
        return out

    def relu(inp):
        out = inp + ".relu"
        g.add("Relu", [inp], [out])
        return out

    assert model.version == 1, "graph export covers the v1 / v1.5 layout"
    h = relu(bn(model.stem_bn, conv(model.stem, x)))
    if model.first_pool:
        g.add("MaxPool", [h], ["pool.out"], kernel_shape=[3, 3], strides=[2, 2], pads=[1, 1, 1, 1])
        h = "pool.out"
    for bi, blk in enumerate(model.blocks):
        sc = h
        if blk.proj is not None:
            sc = bn(blk.proj_bn, conv(blk.proj, h))
        y = h
        for i, (c, b) in enumerate(zip(blk.convs, blk.bns)):
            y = bn(b, conv(c, y))
            if i < len(blk.convs) - 1:
                y = relu(y)
        g.add("Add", [y, sc], ["block%d.sum" % bi])
        h = relu("block%d.sum" % bi)
    g.add("GlobalAveragePool", [h], ["gap.out"])
    g.add("Flatten", ["gap.out"], ["flat.out"], axis=1)
    w = g.add_initializer("fc.weight", model.fc.weight.detach().float().numpy())
    b = g.add_initializer("fc.bias", model.fc.bias.detach().float().numpy())
    g.add("Gemm", ["flat.out", w, b], ["logits"], transB=1)
    g.add_output("logits")
    return g
