"""More ONNX operators for the graph executor: comparisons and logic, selection, the rest of the activations and
reductions, shape and data movement, transposed convolution, instance normalisation, resizing.

The reference's TensorFlow visitor maps 69 ONNX operators and its PyTorch visitor 32
(deep500/frameworks/tensorflow/tf_visitor_impl.py, frameworks/pytorch/pytorch_visitor.py); with this mix-in the
executor here runs 106 (the loss and gradient-exchange extensions included).  Each method reads its inputs with ``self._in(op, k)`` (None for an absent optional input) and
attributes from ``op.attrs`` with the ONNX defaults; semantics follow the ONNX operator specification, opset 13,
with the attribute forms of older opsets (``axes`` / ``split`` / ``pads`` as attributes) accepted as well.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.nn.functional as F

_ONNX_DTYPES = {1: torch.float32, 2: torch.uint8, 3: torch.int8, 5: torch.int16, 6: torch.int32, 7: torch.int64,
                9: torch.bool, 10: torch.float16, 11: torch.float64, 16: torch.bfloat16}


def _ints(t):
    """A tensor or list of integers as a python list (shape-like inputs arrive as tensors from opset 13 on)."""
    if t is None:
        return None
    if isinstance(t, torch.Tensor):
        return [int(v) for v in t.flatten().tolist()]
    return [int(v) for v in np.asarray(t).flatten().tolist()]


class MoreOperators:
    def _outs(self, op, values):
        for name, v in zip(op.outputs, values):
            if name != "":
                self.v[name] = v

    def _axes(self, op, k=1):
        """Reduction / squeeze axes: input ``k`` (opset 13) or the ``axes`` attribute (older)."""
        t = self._in(op, k)
        return _ints(t) if t is not None else op.attrs.get("axes")

    # ---- comparisons, logic, selection --------------------------------------------------------------------------------
    def visit_equal(self, op, g): self._out(op, self._in(op, 0) == self._in(op, 1))
    def visit_greater(self, op, g): self._out(op, self._in(op, 0) > self._in(op, 1))
    def visit_greaterorequal(self, op, g): self._out(op, self._in(op, 0) >= self._in(op, 1))
    def visit_less(self, op, g): self._out(op, self._in(op, 0) < self._in(op, 1))
    def visit_lessorequal(self, op, g): self._out(op, self._in(op, 0) <= self._in(op, 1))
    def visit_and(self, op, g): self._out(op, self._in(op, 0) & self._in(op, 1))
    def visit_or(self, op, g): self._out(op, self._in(op, 0) | self._in(op, 1))
    def visit_xor(self, op, g): self._out(op, self._in(op, 0) ^ self._in(op, 1))
    def visit_not(self, op, g): self._out(op, ~self._in(op, 0))
    def visit_where(self, op, g): self._out(op, torch.where(self._in(op, 0), self._in(op, 1), self._in(op, 2)))
    def visit_isnan(self, op, g): self._out(op, torch.isnan(self._in(op, 0)))

    def visit_max(self, op, g):
        y = self.v[op.inputs[0]]
        for i in op.inputs[1:]:
            y = torch.maximum(y, self.v[i])
        self._out(op, y)

    def visit_min(self, op, g):
        y = self.v[op.inputs[0]]
        for i in op.inputs[1:]:
            y = torch.minimum(y, self.v[i])
        self._out(op, y)

    def visit_mean(self, op, g): self._out(op, sum(self.v[i] for i in op.inputs) / len(op.inputs))

    # ---- unary maths and activations -----------------------------------------------------------------------------------
    def visit_floor(self, op, g): self._out(op, torch.floor(self._in(op, 0)))
    def visit_ceil(self, op, g): self._out(op, torch.ceil(self._in(op, 0)))
    def visit_round(self, op, g): self._out(op, torch.round(self._in(op, 0)))          # half to even, as ONNX
    def visit_sign(self, op, g): self._out(op, torch.sign(self._in(op, 0)))
    def visit_reciprocal(self, op, g): self._out(op, torch.reciprocal(self._in(op, 0)))
    def visit_erf(self, op, g): self._out(op, torch.erf(self._in(op, 0)))
    def visit_sin(self, op, g): self._out(op, torch.sin(self._in(op, 0)))
    def visit_cos(self, op, g): self._out(op, torch.cos(self._in(op, 0)))
    def visit_softplus(self, op, g): self._out(op, F.softplus(self._in(op, 0)))
    def visit_softsign(self, op, g): self._out(op, F.softsign(self._in(op, 0)))
    def visit_elu(self, op, g): self._out(op, F.elu(self._in(op, 0), op.attrs.get("alpha", 1.0)))

    def visit_selu(self, op, g):
        a, s = op.attrs.get("alpha", 1.67326319217681884765625), op.attrs.get("gamma", 1.05070102214813232421875)
        x = self._in(op, 0)
        self._out(op, s * torch.where(x > 0, x, a * (torch.exp(x) - 1)))

    def visit_hardsigmoid(self, op, g):
        self._out(op, (op.attrs.get("alpha", 0.2) * self._in(op, 0) + op.attrs.get("beta", 0.5)).clamp(0, 1))

    def visit_prelu(self, op, g):
        x, slope = self._in(op, 0), self._in(op, 1)
        self._out(op, torch.where(x >= 0, x, x * slope))

    def visit_thresholdedrelu(self, op, g):
        x = self._in(op, 0)
        self._out(op, torch.where(x > op.attrs.get("alpha", 1.0), x, torch.zeros_like(x)))

    def visit_cast(self, op, g): self._out(op, self._in(op, 0).to(_ONNX_DTYPES[int(op.attrs["to"])]))

    # ---- the experimental operators of early ONNX releases (the reference has classes for them) -----------------------
    def visit_affine(self, op, g): self._out(op, op.attrs.get("alpha", 1.0) * self._in(op, 0) + op.attrs.get("beta", 0.0))

    def visit_scale(self, op, g): self._out(op, self._in(op, 0) * op.attrs.get("scale", 1.0))

    def visit_scaledtanh(self, op, g):
        self._out(op, op.attrs.get("alpha", 1.0) * torch.tanh(op.attrs.get("beta", 1.0) * self._in(op, 0)))

    def visit_parametricsoftplus(self, op, g):
        a, b = op.attrs.get("alpha", 1.0), op.attrs.get("beta", 1.0)
        self._out(op, a * torch.nn.functional.softplus(b * self._in(op, 0)))

    def visit_imagescaler(self, op, g):
        x = self._in(op, 0)
        y = x * op.attrs.get("scale", 1.0)
        bias = op.attrs.get("bias")
        if bias is not None:
            y = y + torch.as_tensor(np.asarray(bias, dtype=np.float32), device=x.device).to(x.dtype).view(1, -1, 1, 1)
        self._out(op, y)

    def visit_crop(self, op, g):
        x = self._in(op, 0)
        left, top, right, bottom = [int(v) for v in op.attrs["border"]]
        scale = op.attrs.get("scale")
        if scale is not None:                            # the size of the crop instead of its right / bottom border
            h, w = int(scale[0]), int(scale[1])
            self._out(op, x[..., top:top + h, left:left + w])
        else:
            self._out(op, x[..., top:x.shape[-2] - bottom, left:x.shape[-1] - right])

    def _device(self):
        return next(self.net.parameters()).device

    def _fill_shape(self, op):
        if int(op.attrs.get("input_as_shape", 0)):
            shape = _ints(self._in(op, 0))
        elif op.inputs and op.inputs[0] != "":
            shape = list(self._in(op, 0).shape)
        else:
            shape = [int(v) for v in (op.attrs.get("shape") or [])]
        return shape + [int(v) for v in (op.attrs.get("extra_shape") or [])]

    def visit_constantfill(self, op, g):
        dt = _ONNX_DTYPES[int(op.attrs.get("dtype", 1))]
        self._out(op, torch.full(self._fill_shape(op), op.attrs.get("value", 0.0), dtype=dt, device=self._device()))

    def visit_giventensorfill(self, op, g):
        v = torch.as_tensor(np.asarray(op.attrs.get("values") or [], dtype=np.float32), device=self._device())
        self._out(op, v.reshape(self._fill_shape(op)))

    # ---- reductions ---------------------------------------------------------------------------------------------------
    def _reduce(self, op, fn):
        x, axes = self._in(op, 0), self._axes(op)
        keep = bool(op.attrs.get("keepdims", 1))
        if axes is None:
            axes = list(range(x.dim()))
        self._out(op, fn(x, [int(a) for a in axes], keep))

    def visit_reducemax(self, op, g): self._reduce(op, lambda x, a, k: torch.amax(x, dim=a, keepdim=k))
    def visit_reducemin(self, op, g): self._reduce(op, lambda x, a, k: torch.amin(x, dim=a, keepdim=k))
    def visit_reduceprod(self, op, g):
        def prod(x, axes, keep):
            for a in sorted((a % x.dim() for a in axes), reverse=True):
                x = x.prod(dim=a, keepdim=keep)
            return x
        self._reduce(op, prod)
    def visit_reducel1(self, op, g): self._reduce(op, lambda x, a, k: x.abs().sum(dim=a, keepdim=k))
    def visit_reducel2(self, op, g): self._reduce(op, lambda x, a, k: x.square().sum(dim=a, keepdim=k).sqrt())
    def visit_reducesumsquare(self, op, g): self._reduce(op, lambda x, a, k: x.square().sum(dim=a, keepdim=k))
    def visit_reducelogsumexp(self, op, g): self._reduce(op, lambda x, a, k: torch.logsumexp(x, dim=a, keepdim=k))

    def visit_argmax(self, op, g):
        self._out(op, torch.argmax(self._in(op, 0), dim=op.attrs.get("axis", 0), keepdim=bool(op.attrs.get("keepdims", 1))))

    def visit_argmin(self, op, g):
        self._out(op, torch.argmin(self._in(op, 0), dim=op.attrs.get("axis", 0), keepdim=bool(op.attrs.get("keepdims", 1))))

    def visit_topk(self, op, g):
        k = _ints(self._in(op, 1))[0] if self._in(op, 1) is not None else int(op.attrs["k"])
        vals, idx = torch.topk(self._in(op, 0), k, dim=op.attrs.get("axis", -1), largest=bool(op.attrs.get("largest", 1)),
                               sorted=bool(op.attrs.get("sorted", 1)))
        self._outs(op, [vals, idx])

    def visit_cumsum(self, op, g):
        x, axis = self._in(op, 0), _ints(self._in(op, 1))[0]
        rev, excl = bool(op.attrs.get("reverse", 0)), bool(op.attrs.get("exclusive", 0))
        if rev:
            x = x.flip(axis)
        y = torch.cumsum(x, axis)
        if excl:
            y = y - x
        self._out(op, y.flip(axis) if rev else y)

    # ---- shapes and data movement -----------------------------------------------------------------------------------------
    def visit_shape(self, op, g): self._out(op, torch.tensor(list(self._in(op, 0).shape), dtype=torch.int64))
    def visit_size(self, op, g): self._out(op, torch.tensor(self._in(op, 0).numel(), dtype=torch.int64))
    def visit_expand(self, op, g):
        x, shape = self._in(op, 0), _ints(self._in(op, 1))
        self._out(op, x * torch.ones(shape, dtype=x.dtype, device=x.device))                  # numpy-style broadcast
    def visit_tile(self, op, g): self._out(op, self._in(op, 0).repeat(*_ints(self._in(op, 1))))
    def visit_gather(self, op, g):
        x, idx = self._in(op, 0), self._in(op, 1).long()
        axis = op.attrs.get("axis", 0) % x.dim()
        idx = torch.where(idx < 0, idx + x.shape[axis], idx)
        y = torch.index_select(x, axis, idx.flatten())
        self._out(op, y.reshape(x.shape[:axis] + idx.shape + x.shape[axis + 1:]))

    def visit_slice(self, op, g):
        x = self._in(op, 0)
        starts = _ints(self._in(op, 1)) if self._in(op, 1) is not None else op.attrs["starts"]
        ends = _ints(self._in(op, 2)) if self._in(op, 2) is not None else op.attrs["ends"]
        axes = _ints(self._in(op, 3)) if self._in(op, 3) is not None else op.attrs.get("axes", list(range(len(starts))))
        steps = _ints(self._in(op, 4)) if self._in(op, 4) is not None else [1] * len(starts)
        index = [slice(None)] * x.dim()
        for s, e, a, st in zip(starts, ends, axes, steps):
            if st <= 0:
                raise NotImplementedError("Slice with a non-positive step")
            n = x.shape[a]
            index[a] = slice(max(s + n, 0) if s < 0 else min(s, n), max(e + n, 0) if e < 0 else min(e, n), st)
        self._out(op, x[tuple(index)])

    def visit_split(self, op, g):
        x, axis = self._in(op, 0), op.attrs.get("axis", 0)
        sizes = _ints(self._in(op, 1)) if self._in(op, 1) is not None else op.attrs.get("split")
        if sizes is None:
            sizes = [x.shape[axis] // len(op.outputs)] * len(op.outputs)
        self._outs(op, torch.split(x, sizes, dim=axis))

    def visit_depthtospace(self, op, g):
        x, b = self._in(op, 0), int(op.attrs["blocksize"])
        n, c, h, w = x.shape
        if op.attrs.get("mode", "DCR") == "DCR":
            y = x.reshape(n, b, b, c // (b * b), h, w).permute(0, 3, 4, 1, 5, 2)
        else:
            y = x.reshape(n, c // (b * b), b, b, h, w).permute(0, 1, 4, 2, 5, 3)
        self._out(op, y.reshape(n, c // (b * b), h * b, w * b))

    def visit_spacetodepth(self, op, g):
        x, b = self._in(op, 0), int(op.attrs["blocksize"])
        n, c, h, w = x.shape
        y = x.reshape(n, c, h // b, b, w // b, b).permute(0, 3, 5, 1, 2, 4)
        self._out(op, y.reshape(n, c * b * b, h // b, w // b))

    def visit_constantofshape(self, op, g):
        v = op.attrs.get("value")
        v = torch.as_tensor(np.asarray(v)).flatten()[0] if v is not None else torch.tensor(0.0)
        self._out(op, torch.full(_ints(self._in(op, 0)), v.item(), dtype=v.dtype))

    def visit_range(self, op, g):
        s, e, d = (self._in(op, k) for k in range(3))
        self._out(op, torch.arange(s.item(), e.item(), d.item(), dtype=s.dtype))

    def visit_onehot(self, op, g):
        idx, depth, values = self._in(op, 0).long(), int(_ints(self._in(op, 1))[0]), self._in(op, 2)
        idx = torch.where(idx < 0, idx + depth, idx)
        hot = F.one_hot(idx, depth).movedim(-1, op.attrs.get("axis", -1))
        self._out(op, torch.where(hot.bool(), values[1], values[0]))

    # ---- layers -----------------------------------------------------------------------------------------------------------
    def visit_convtranspose(self, op, g):
        x, w, b = self._in(op, 0), self._in(op, 1), self._in(op, 2)
        a = op.attrs
        self._out(op, F.conv_transpose2d(x, w, b, stride=tuple(a.get("strides", [1, 1])), padding=tuple(a.get("pads", [0, 0, 0, 0])[:2]),
                                         output_padding=tuple(a.get("output_padding", [0, 0])), groups=int(a.get("group", 1)),
                                         dilation=tuple(a.get("dilations", [1, 1]))))

    def visit_instancenormalization(self, op, g):
        x, s, b = self._in(op, 0), self._in(op, 1), self._in(op, 2)
        self._out(op, F.instance_norm(x, weight=s, bias=b, eps=op.attrs.get("epsilon", 1e-5)))

    def visit_globalmaxpool(self, op, g): self._out(op, torch.amax(self._in(op, 0), dim=(2, 3), keepdim=True))

    def visit_lpnormalization(self, op, g):
        self._out(op, F.normalize(self._in(op, 0), p=float(op.attrs.get("p", 2)), dim=op.attrs.get("axis", -1), eps=0.0))

    def visit_resize(self, op, g):
        x = self._in(op, 0)
        scales, sizes = self._in(op, 2), self._in(op, 3)
        mode = {"nearest": "nearest", "linear": "bilinear", "cubic": "bicubic"}[op.attrs.get("mode", "nearest")]
        kw = {} if mode == "nearest" else {"align_corners": op.attrs.get("coordinate_transformation_mode") == "align_corners"}
        if sizes is not None and sizes.numel():
            self._out(op, F.interpolate(x, size=_ints(sizes)[2:], mode=mode, **kw))
        else:
            self._out(op, F.interpolate(x, scale_factor=[float(v) for v in scales.flatten().tolist()[2:]], mode=mode, **kw))

    def visit_upsample(self, op, g):
        sc = self._in(op, 1)
        sc = [float(v) for v in sc.flatten().tolist()] if sc is not None else [float(v) for v in op.attrs["scales"]]
        self._out(op, F.interpolate(self._in(op, 0), scale_factor=sc[2:], mode=op.attrs.get("mode", "nearest")))

    def visit_lstm(self, op, g):
        """ONNX LSTM, forward direction, zero initial state, full-length sequences: runs on this package's LSTM layer
        (tensor-core projections and the native time loop on a GPU).  ONNX orders the gates i, o, f, c and splits the
        bias into an input and a recurrent half; the layer wants i, f, g, o and their sum."""
        from ..ops.lstm import lstm_layer
        x, w, r, b = (self._in(op, k) for k in range(4))
        if op.attrs.get("direction", "forward") != "forward" or any(self._in(op, k) is not None for k in (4, 5, 6, 7)):
            raise NotImplementedError("LSTM: only the forward direction with zero initial state and no sequence_lens")
        if op.attrs.get("layout", 0) != 0:
            raise NotImplementedError("LSTM: batch-major layout")
        h = r.shape[-1]
        order = torch.cat([torch.arange(0, h), torch.arange(2 * h, 3 * h), torch.arange(3 * h, 4 * h), torch.arange(h, 2 * h)]).to(w.device)
        w_ih, w_hh = w[0].index_select(0, order), r[0].index_select(0, order)
        bias = (b[0, :4 * h] + b[0, 4 * h:]).index_select(0, order) if b is not None else torch.zeros(4 * h, device=w.device)
        y = lstm_layer(x, w_ih.to(x.dtype).contiguous(), w_hh.to(x.dtype).contiguous(), bias.float())      # [T, B, H]
        outs = [y.unsqueeze(1), y[-1].unsqueeze(0)]
        if len(op.outputs) > 2 and op.outputs[2] != "":
            raise NotImplementedError("LSTM: the final cell state is not an output of the layer")
        self._outs(op, outs)

