"""Run a ``Graph`` on the CPU oracles only (numpy and the compiled C++ operators), forward and backward.

The counterpart of the reference's own framework-free back end
(deep500/frameworks/reference/reference_network.py, reference_graph_executor.py:34-47 and the two
build-graph visitors over its python and C++ operators): a topological forward pass that keeps every
intermediate value, and a reverse pass that hands each operator its output gradient.  Nothing here touches
PyTorch or a GPU, which is the point: it is the independent check for the native executor
(``graph.executor.GraphNetwork``) and for hand-written kernels.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import numpy as np

from ..ref import cpp_ops as CPP
from ..ref import numpy_ops as NP
from .ir import Graph, Operation


def _pads(op: Operation) -> int:
    p = op.attrs.get("pads", [0, 0, 0, 0])
    if len(set(p)) > 1:
        raise NotImplementedError("%s: asymmetric padding %s" % (op.name, p))
    return int(p[0]) if p else 0


class ReferenceGraphExecutor:
    """``inference(feeds)`` returns the graph outputs; ``inference_and_backprop(feeds, loss)`` also fills
    ``gradients`` (by tensor name) for every initializer the loss depends on.  ``use_cpp`` picks the compiled
    operators where both kinds exist."""

    def __init__(self, graph: Graph, use_cpp: bool = True, training: bool = True):
        self.graph, self.use_cpp, self.training = graph, use_cpp, training
        self.values: Dict[str, np.ndarray] = {}
        self.gradients: Dict[str, np.ndarray] = {}
        self._saved: Dict[str, tuple] = {}
        self.order = graph.topological()

    # ---- forward ------------------------------------------------------------------------------------------------
    def inference(self, feeds: Dict[str, np.ndarray]) -> List[np.ndarray]:
        v = self.values = {k: np.asarray(a) for k, a in self.graph.initializers.items()}
        v.update({k: np.asarray(a) for k, a in feeds.items()})
        for op in self.order:
            fn = getattr(self, "_fwd_" + op.op_type.lower(), None)
            if fn is None:
                raise NotImplementedError("reference executor: no forward for %s" % op.op_type)
            out = fn(op, [v[i] if i else None for i in op.inputs])
            for name, val in zip(op.outputs, out if isinstance(out, (tuple, list)) else [out]):
                v[name] = val
        return [v[o] for o in self.graph.outputs]

    def _fwd_conv(self, op, x):
        stride = int(op.attrs.get("strides", [1, 1])[0])
        mod = CPP if self.use_cpp else NP
        y = mod.conv2d(x[0].astype(np.float32), x[1].astype(np.float32), stride, _pads(op))
        if len(x) > 2 and x[2] is not None:
            y = y + x[2].reshape(1, -1, 1, 1)
        return y

    def _fwd_batchnormalization(self, op, x):
        eps = float(op.attrs.get("epsilon", 1e-5))
        if self.training:
            mod = CPP if self.use_cpp else NP
            y, _, _, mean, invstd = mod.batchnorm_training(x[0], x[1], x[2], x[3], x[4],
                                                           1.0 - float(op.attrs.get("momentum", 0.9)), eps)
            self._saved[op.name] = (mean, invstd)
            return y
        return (CPP if self.use_cpp else NP).batchnorm_inference(x[0], x[1], x[2], x[3], x[4], eps)

    def _fwd_relu(self, op, x): return (CPP.relu if self.use_cpp else NP.relu)(x[0])
    def _fwd_add(self, op, x): return x[0] + x[1]
    def _fwd_sum(self, op, x): return CPP.sum_n(x) if self.use_cpp and all(a.shape == x[0].shape for a in x) else sum(x)
    def _fwd_identity(self, op, x): return x[0]
    def _fwd_flatten(self, op, x): return x[0].reshape(x[0].shape[0], -1)
    def _fwd_reshape(self, op, x): return x[0].reshape(op.attrs["shape"])
    def _fwd_matmul(self, op, x): return CPP.matmul(x[0], x[1]) if self.use_cpp and x[0].ndim == 2 else x[0] @ x[1]
    def _fwd_softmax(self, op, x): return CPP.softmax(x[0]) if self.use_cpp and x[0].ndim == 2 else NP.softmax(x[0])
    def _fwd_globalaveragepool(self, op, x): return x[0].mean((2, 3), keepdims=True)

    def _fwd_maxpool(self, op, x):
        k, s = int(op.attrs["kernel_shape"][0]), int(op.attrs.get("strides", [1, 1])[0])
        return (CPP if self.use_cpp else NP).maxpool(x[0], k, s, _pads(op))

    def _fwd_averagepool(self, op, x):
        k, s = int(op.attrs["kernel_shape"][0]), int(op.attrs.get("strides", [1, 1])[0])
        if self.use_cpp:
            return CPP.avgpool(x[0], k, s, _pads(op), bool(op.attrs.get("count_include_pad", 0)))
        return NP.averagepool(x[0], k, s, _pads(op))

    def _fwd_gemm(self, op, x):
        a = op.attrs
        c = x[2] if len(x) > 2 else None
        y = (CPP if self.use_cpp else NP).gemm(x[0], x[1], None, float(a.get("alpha", 1.0)), 0.0,
                                               bool(a.get("transA", 0)), bool(a.get("transB", 0)))
        return y + float(a.get("beta", 1.0)) * c if c is not None else y

    def _fwd_softmaxcrossentropy(self, op, x):
        loss, dlogits = NP.softmax_cross_entropy(x[0].astype(np.float64), x[1].astype(np.int64))
        self._saved[op.name] = (dlogits,)
        return np.asarray(loss)

    def _fwd_meansquarederror(self, op, x): return np.asarray(np.mean((x[0] - x[1]) ** 2))

    # ---- backward -----------------------------------------------------------------------------------------------
    def inference_and_backprop(self, feeds: Dict[str, np.ndarray], loss: Optional[str] = None) -> List[np.ndarray]:
        outs = self.inference(feeds)
        loss = loss or self.graph.outputs[-1]
        g: Dict[str, np.ndarray] = {loss: np.ones_like(self.values[loss], dtype=np.float64)}
        for op in reversed(self.order):
            if not any(o in g for o in op.outputs):
                continue
            fn = getattr(self, "_bwd_" + op.op_type.lower(), None)
            if fn is None:
                raise NotImplementedError("reference executor: no backward for %s" % op.op_type)
            ins = [self.values[i] if i else None for i in op.inputs]
            grads = fn(op, ins, g[op.outputs[0]])
            for name, gi in zip(op.inputs, grads):
                if gi is None or not name:
                    continue
                g[name] = g[name] + gi if name in g else gi
        self.gradients = {k: v for k, v in g.items() if k in self.graph.initializers}
        return outs

    def _bwd_conv(self, op, x, dy):
        stride = int(op.attrs.get("strides", [1, 1])[0])
        mod = CPP if self.use_cpp else NP
        fn = mod.conv2d_grads if self.use_cpp else mod.conv2d_grad
        dx, dw = fn(x[0].astype(np.float32), x[1].astype(np.float32), dy.astype(np.float32), stride, _pads(op))
        db = dy.sum((0, 2, 3)) if len(x) > 2 and x[2] is not None else None
        return [dx, dw, db]

    def _bwd_batchnormalization(self, op, x, dy):
        if self.training:
            mean, invstd = self._saved[op.name]
            dx, dg, db = (CPP if self.use_cpp else NP).batchnorm_training_grad(x[0], x[1], mean, invstd, dy)
        else:
            dx, dg, db = CPP.batchnorm_inference_grad(x[0], x[1], x[3], x[4], dy, float(op.attrs.get("epsilon", 1e-5)))
        return [dx, dg, db, None, None]

    def _bwd_relu(self, op, x, dy): return [(CPP if self.use_cpp else NP).relu_grad(x[0], dy)]
    def _bwd_add(self, op, x, dy): return [_unbroadcast(dy, x[0].shape), _unbroadcast(dy, x[1].shape)]
    def _bwd_sum(self, op, x, dy): return [_unbroadcast(dy, a.shape) for a in x]
    def _bwd_identity(self, op, x, dy): return [dy]
    def _bwd_flatten(self, op, x, dy): return [dy.reshape(x[0].shape)]
    def _bwd_reshape(self, op, x, dy): return [dy.reshape(x[0].shape)] + [None] * (len(x) - 1)
    def _bwd_matmul(self, op, x, dy): return list(CPP.matmul_grad(x[0], x[1], dy)) if x[0].ndim == 2 else [dy @ x[1].T, x[0].T @ dy]
    def _bwd_softmax(self, op, x, dy): return [CPP.softmax_grad(self.values[op.outputs[0]], dy)]
    def _bwd_globalaveragepool(self, op, x, dy): return [CPP.global_avgpool_grad(dy.reshape(dy.shape[0], dy.shape[1]), x[0].shape)]

    def _bwd_maxpool(self, op, x, dy):
        k, s = int(op.attrs["kernel_shape"][0]), int(op.attrs.get("strides", [1, 1])[0])
        return [CPP.maxpool_grad(x[0], dy, k, s, _pads(op))]

    def _bwd_averagepool(self, op, x, dy):
        k, s = int(op.attrs["kernel_shape"][0]), int(op.attrs.get("strides", [1, 1])[0])
        return [CPP.avgpool_grad(dy, x[0].shape, k, s, _pads(op), bool(op.attrs.get("count_include_pad", 0)))]

    def _bwd_gemm(self, op, x, dy):
        a = op.attrs
        da, db, dc = CPP.gemm_grad(x[0], x[1], dy, float(a.get("alpha", 1.0)), float(a.get("beta", 1.0)),
                                   bool(a.get("transA", 0)), bool(a.get("transB", 0)))
        out = [da, db]
        if len(x) > 2:
            out.append(_unbroadcast(dc, x[2].shape))
        return out

    def _bwd_softmaxcrossentropy(self, op, x, dy):
        (dlogits,) = self._saved[op.name]
        return [dlogits * dy, None]

    def _bwd_meansquarederror(self, op, x, dy):
        d = 2.0 * (x[0] - x[1]) / x[0].size * dy
        return [d, -d]


def _unbroadcast(g: np.ndarray, shape: Tuple[int, ...]) -> np.ndarray:
    """Sum a gradient over the axes numpy broadcast to reach ``g.shape`` from ``shape``."""
    g = np.asarray(g)
    while g.ndim > len(shape):
        g = g.sum(0)
    for ax, n in enumerate(shape):
        if n == 1 and g.shape[ax] != 1:
            g = g.sum(ax, keepdims=True)
    return g.reshape(shape)
