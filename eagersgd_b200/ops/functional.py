"""Autograd functions over the hand-written sm_100a kernels (NHWC bf16 activations).

Activations are 4-D ``channels_last`` tensors, i.e. ``[N, H, W, C]`` in memory,
which makes a 1x1 convolution a plain ``[N*H*W, Cin] x [Cout, Cin]^T`` GEMM on
the tcgen05 tensor cores, with the batch-norm statistics accumulated in the GEMM
epilogue.  On CPU tensors every function falls back to the same mathematics in
PyTorch, which is what the CPU tests and oracles use.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import contextlib

import os

import torch
import torch.nn.functional as F

from ..parallel import _native as N
from .gemm import gemm

BN_EPS = 1e-5


def _lib():
    lib = N.cuda()
    if not getattr(lib, "_nn_bound", False):
        vp, i32, i64, f32 = C.c_void_p, C.c_int, C.c_int64, C.c_float
        lib.esgd_bn_stats.argtypes = [vp, i64, i32, vp, vp, vp]
        lib.esgd_bn_finalize.argtypes = [vp] * 10 + [i32, i64, f32, f32, vp]
        lib.esgd_bn_apply.argtypes = [vp, vp, vp, vp, vp, i64, i32, i32, vp]
        lib.esgd_bn_bwd_reduce.argtypes = [vp] * 7 + [i64, i32, i32, vp, vp, vp]
        lib.esgd_bn_bwd_apply.argtypes = [vp] * 12 + [i64, i32, i32, vp]
        lib.esgd_softmax_ce.argtypes = [vp, i32, vp, i32, i32, i32, f32, vp, vp, vp, vp]
        lib.esgd_maxpool3x3s2_fwd.argtypes = [vp, vp, vp, i32, i32, i32, i32, vp]
        lib.esgd_subsample2_fwd.argtypes = [vp, vp, i32, i32, i32, i32, vp]
        lib.esgd_subsample2_bwd.argtypes = [vp, vp, i32, i32, i32, i32, vp]
        lib.esgd_maxpool3x3s2_bwd.argtypes = [vp, vp, vp, i32, i32, i32, i32, vp]
        lib.esgd_avgpool_fwd.argtypes = [vp, vp, i32, i32, i32, vp]
        lib.esgd_avgpool_bwd.argtypes = [vp, vp, i32, i32, i32, vp]
        lib.esgd_conv2d_fwd.argtypes = [vp, vp, vp] + [i32] * 10 + [vp, vp, vp, vp]
        lib.esgd_conv2d_fwd_ex.argtypes = [vp, vp, vp] + [i32] * 11 + [i64, i64, i64, i32, vp, vp, vp, vp]
        lib.esgd_im2col_small_c.argtypes = [vp, vp] + [i32] * 10 + [vp]
        lib.esgd_conv2d_wgrad.argtypes = [vp, vp, vp] + [i32] * 9 + [vp, vp]
        lib.esgd_conv2d_wgrad_halo.argtypes = [vp, vp, vp] + [i32] * 8 + [vp, vp]
        lib._nn_bound = True
    return lib


def _stream(t: torch.Tensor):
    return torch.cuda.current_stream(t.device).cuda_stream


def _ck(rc: int, what: str):
    if rc != 0:
        raise RuntimeError("%s failed with code %d" % (what, rc))


def _ptr(t: Optional[torch.Tensor]):
    return t.data_ptr() if t is not None else None


def nhwc_2d(x: torch.Tensor) -> torch.Tensor:
    """[N, C, H, W] channels_last -> contiguous [N*H*W, C] view (no copy when already NHWC)."""
    n, c, h, w = x.shape
    return x.permute(0, 2, 3, 1).contiguous().view(n * h * w, c)


def from_2d(y2d: torch.Tensor, n: int, h: int, w: int) -> torch.Tensor:
    return y2d.view(n, h, w, y2d.shape[1]).permute(0, 3, 1, 2)


_reference_only = False


class _ZeroArena:
    """One fp32 buffer cleared by a single memset at the start of a training step, from which the operators take
    their zero-initialised scratch (statistics accumulators, fp32 weight-gradient accumulators) instead of each
    launching a fill kernel of its own: about 180 fills per ResNet-50 step become one.  Only active inside
    ``zero_arena()``; slices must not outlive the step (the users here consume them at once)."""

    def __init__(self):
        self.buf = None
        self.off = 0
        self.dirty = 0          # floats handed out in any step so far: the prefix that has to be cleared again
        self.cap = 0
        self.device = None
        self.active = False

    def begin(self, device, numel):
        if self.buf is not None and (self.buf.device != device or self.buf.numel() < numel):
            self.buf, self.dirty = None, 0
        self.device, self.cap = device, numel
        if self.buf is not None and self.dirty > 0:
            self.buf[:self.dirty].zero_()                # one memset over what earlier steps used
        self.off = 0
        self.active = True

    def take(self, shape, device):
        n = 1
        for d in shape:
            n *= int(d)
        n_al = (n + 63) // 64 * 64                      # keep every slice 256-byte aligned
        if not self.active or self.device != device or self.off + n_al > self.cap:
            return torch.zeros(shape, dtype=torch.float32, device=device)
        if self.buf is None:                             # first use: models that never ask pay nothing
            self.buf = torch.zeros(self.cap, dtype=torch.float32, device=device)
        out = self.buf[self.off:self.off + n].view(shape)
        self.off += n_al
        self.dirty = max(self.dirty, self.off)
        return out


_arena = _ZeroArena()


@contextlib.contextmanager
def zero_arena(device, numel: int):
    """Serve the operators' zeroed fp32 scratch from one buffer of ``numel`` floats for the duration of a step."""
    _arena.begin(torch.device(device), numel)
    try:
        yield
    finally:
        _arena.active = False


def zeros_f32(shape, device):
    return _arena.take(tuple(shape), torch.device(device) if not isinstance(device, torch.device) else device)


class reference_ops:
    """Context manager: run every op through its PyTorch restatement (the test oracle)."""

    def __enter__(self):
        global _reference_only
        self._prev, _reference_only = _reference_only, True

    def __exit__(self, *a):
        global _reference_only
        _reference_only = self._prev


def native(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16 and not _reference_only


# --------------------------------------------------------------------------- 1x1 convolution / dense
def wgrad_splits(pixels: int, cout: int, cin: int, sms: int = 148) -> int:
    """Split-K factor of a weight-gradient GEMM (K = pixels): about one wave of tiles.  Each split adds a
    full [Cout, Cin] partial result with atomics, so large filter banks take few splits."""
    bn = 64 if cin <= 64 else (128 if cin <= 128 else 256)
    out_tiles = -(-cout // 128) * -(-cin // bn)
    return max(2, min(-(-sms // out_tiles), max(1, (pixels // 64) // 8)))


class _Conv1x1(torch.autograd.Function):
    """y = x (*) w for a 1x1 kernel; optionally also returns per-channel sum / sum-of-squares of y.

    With ``tap_input`` the input is returned as a last output, too.  A residual block takes its shortcut
    from that output instead of from ``x`` itself: backward then receives the shortcut's gradient together
    with dy and adds it in the epilogue of the data-gradient GEMM, instead of autograd summing the two
    branches of ``x`` with a separate pass over the tensor."""

    @staticmethod
    def forward(ctx, x, w, want_stats: bool, tap_input: bool = False):
        n, cin, h, wd = x.shape
        cout = w.shape[0]
        x2d = nhwc_2d(x)
        w2d = w.reshape(cout, cin)
        stats = zeros_f32((2, cout), x.device) if want_stats else None
        y2d = gemm(x2d, w2d, col_sum=stats[0] if want_stats else None, col_sqsum=stats[1] if want_stats else None)
        ctx.save_for_backward(x2d, w2d)
        ctx.dims = (n, h, wd, cin, cout, w.shape)
        ctx.mark_non_differentiable(*( [stats] if want_stats else []))
        ctx.layout = (want_stats, tap_input)
        ctx.set_materialize_grads(False)       # an unused tap must not cost a tensor of zeros
        y = from_2d(y2d, n, h, wd)
        outs = (y,) + ((stats,) if want_stats else ()) + ((x.view_as(x),) if tap_input else ())
        return outs if len(outs) > 1 else y

    @staticmethod
    def backward(ctx, dy, *more):
        x2d, w2d = ctx.saved_tensors
        n, h, wd, cin, cout, wshape = ctx.dims
        want_stats, tap_input = ctx.layout
        d_tap = more[-1] if tap_input else None            # gradient that reached the input through the shortcut
        if dy is None:
            return d_tap, None, None, None
        dy2d = nhwc_2d(dy)
        dx = dw = None
        if ctx.needs_input_grad[0]:
            res = nhwc_2d(d_tap.to(torch.bfloat16)) if d_tap is not None else None
            dx = from_2d(gemm(dy2d, w2d, b_kmajor=False, residual=res), n, h, wd)   # [M,Cout] x W[Cout(K),Cin(N)]
        if ctx.needs_input_grad[1]:
            dw32 = gemm(dy2d, x2d, a_kmajor=False, b_kmajor=False, splits=wgrad_splits(dy2d.shape[0], cout, cin),
                        out=zeros_f32((cout, cin), dy2d.device), accumulate=True)            # [Cout, Cin] fp32
            dw = dw32.to(torch.bfloat16).view(wshape)
        return dx, dw, None, None


def conv1x1(x: torch.Tensor, w: torch.Tensor, want_stats: bool = False, tap_input: bool = False):
    """1x1 convolution.  ``tap_input=True`` appends ``x`` itself to the outputs (use it for the shortcut of a
    residual block: the two gradients of ``x`` are then added inside the data-gradient GEMM)."""
    if native(x) and x.shape[1] % 8 == 0 and w.shape[0] % 8 == 0:
        return _Conv1x1.apply(x, w, want_stats, tap_input)
    y = F.conv2d(x, w)
    outs = (y,)
    if want_stats:
        yf = y.float()
        outs += (torch.stack([yf.sum((0, 2, 3)), (yf * yf).sum((0, 2, 3))]).detach(),)
    if tap_input:
        outs += (x,)
    return outs if len(outs) > 1 else y


def _conv_native(x2d_src, w_ohwi, n, h, w, cin, cout, r, s, stride, pad, stats):
    """Launch the implicit-GEMM kernel.  ``x2d_src``: NHWC storage, ``w_ohwi``: [Cout, R, S, Cin] storage."""
    from .gemm import error_flag
    ho, wo = (h + 2 * pad - r) // stride + 1, (w + 2 * pad - s) // stride + 1
    y2d = torch.empty(n * ho * wo, cout, dtype=torch.bfloat16, device=x2d_src.device)
    _ck(_lib().esgd_conv2d_fwd(x2d_src.data_ptr(), w_ohwi.data_ptr(), y2d.data_ptr(), n, h, w, cin, cout, r, s,
                               stride, pad, 0, _ptr(stats[0]) if stats is not None else None,
                               _ptr(stats[1]) if stats is not None else None,
                               error_flag(x2d_src.device).data_ptr(), _stream(x2d_src)), "conv2d")
    return y2d, ho, wo


def _dgrad_stride2(dy, w, n, h, wd, cin, cout):
    """Data gradient of a 3x3 / stride-2 / pad-1 convolution without zero insertion: the four output
    parities (h%2, w%2) are four small convolutions of dy with 1, 2, 2 and 4 of the nine taps
    (dx[2i+a] uses rows r with (a+1-r) even), each written into its strided quarter of dx by TMA."""
    from .gemm import error_flag
    lib = _lib()
    dy2d = nhwc_2d(dy)
    ho, wo = h // 2, wd // 2
    dx2d = torch.empty(n * h * wd, cin, dtype=torch.bfloat16, device=dy.device)
    wt = w.permute(1, 0, 2, 3)                                   # [Cin, Cout, R, S]
    wf = wt.flip(2, 3)                                           # filter indices 2, 1, 0
    taps = {0: [1], 1: [2, 0]}                                   # parity -> filter indices at offsets 0, +1
    sel = {0: slice(1, 2), 1: slice(0, 3, 2)}                    # the same selection on the flipped filter
    esz = dx2d.element_size()
    for a in (0, 1):
        for b in (0, 1):
            ws = wf[:, :, sel[a], sel[b]].contiguous(memory_format=torch.channels_last)
            y_ptr = dx2d.data_ptr() + (a * wd + b) * cin * esz
            _ck(lib.esgd_conv2d_fwd_ex(dy2d.data_ptr(), ws.data_ptr(), y_ptr, n, ho, wo, cout, cin, len(taps[a]),
                                       len(taps[b]), 1, 0, ho, wo, 2 * cin, 2 * wd * cin, h * wd * cin, 0, None, None,
                                       error_flag(dy.device).data_ptr(), _stream(dy)), "strided conv data gradient")
    return from_2d(dx2d, n, h, wd)


class _StemConv(torch.autograd.Function):
    """Convolution with very few input channels (RGB stem): im2col + tensor-core GEMM; the weight
    gradient is one split-K GEMM over the saved columns.  No input gradient (images are leaves)."""

    @staticmethod
    def forward(ctx, x, w, stride, pad, want_stats):
        n, c, h, wd = x.shape
        cout, _, r, s = w.shape
        seg = (s * c + 7) // 8 * 8                                       # one filter row, padded to 16 bytes
        kpad = (r * seg + 63) // 64 * 64
        while kpad % seg:
            kpad += 64
        ho, wo = (h + 2 * pad - r) // stride + 1, (wd + 2 * pad - s) // stride + 1
        col = torch.empty(n * ho * wo, kpad, dtype=torch.bfloat16, device=x.device)
        _ck(_lib().esgd_im2col_small_c(nhwc_2d(x).data_ptr(), col.data_ptr(), n, h, wd, c, r, s, stride, pad, seg,
                                       kpad, _stream(x)), "im2col")
        w2d = torch.zeros(cout, kpad // seg, seg, dtype=torch.bfloat16, device=x.device)
        w2d[:, :r, :s * c] = w.permute(0, 2, 3, 1).reshape(cout, r, s * c)   # [cout][r][(s, c)]
        w2d = w2d.view(cout, kpad)
        stats = zeros_f32((2, cout), x.device) if want_stats else None
        y2d = gemm(col, w2d, col_sum=stats[0] if want_stats else None, col_sqsum=stats[1] if want_stats else None)
        ctx.save_for_backward(col)
        ctx.cfg = (cout, c, r, s, seg)
        y = from_2d(y2d, n, ho, wo)
        if want_stats:
            ctx.mark_non_differentiable(stats)
            return y, stats
        return y

    @staticmethod
    def backward(ctx, dy, *unused):
        (col,) = ctx.saved_tensors
        cout, c, r, s, seg = ctx.cfg
        dy2d = nhwc_2d(dy)
        dw = gemm(dy2d, col, a_kmajor=False, b_kmajor=False, splits=148)        # [Cout, Kpad] fp32
        dw = dw.view(cout, -1, seg)[:, :r, :s * c].reshape(cout, r, s, c).permute(0, 3, 1, 2).to(torch.bfloat16)
        return None, dw, None, None, None


class _ConvKxK(torch.autograd.Function):
    """RxS convolution as an implicit GEMM on the tensor cores (TMA-fed, zero-filled padding)."""

    @staticmethod
    def forward(ctx, x, w, stride, pad, want_stats):
        n, cin, h, wd = x.shape
        cout, _, r, s = w.shape
        w_cl = w.contiguous(memory_format=torch.channels_last)        # [Cout, R, S, Cin] in memory
        # Narrow layers (16 / 32 input channels): the kernel's K blocks are 64 channels wide, so the input and
        # the filters are zero-padded to 64 channels here; the padded input is what backward needs too.
        pin = (-cin) % 64
        if pin:
            x = _pad_channels(x, pin)
            w_f = F.pad(w_cl, (0, 0, 0, 0, 0, pin)).contiguous(memory_format=torch.channels_last)
        else:
            w_f = w_cl
        x2d = nhwc_2d(x)
        stats = zeros_f32((2, cout), x.device) if want_stats else None
        y2d, ho, wo = _conv_native(x2d, w_f, n, h, wd, cin + pin, cout, r, s, stride, pad, stats)
        ctx.save_for_backward(x, w_cl)
        ctx.cfg = (stride, pad)
        y = from_2d(y2d, n, ho, wo)
        if want_stats:
            ctx.mark_non_differentiable(stats)
            return y, stats
        return y

    @staticmethod
    def backward(ctx, dy, *unused):
        x, w = ctx.saved_tensors             # x carries the forward pass's channel padding, w does not
        stride, pad = ctx.cfg
        n, cin_x, h, wd = x.shape
        cout, cin, r, s = w.shape
        dx = dw = None
        dy_cl = dy.contiguous(memory_format=torch.channels_last)
        pout = (-cout) % 64
        if pout:        # the output channels are the reduction dimension of both gradients: pad them with zeros
            dy_cl = _pad_channels(dy_cl, pout)
            w = F.pad(w, (0, 0, 0, 0, 0, 0, 0, pout)).contiguous(memory_format=torch.channels_last)
            cout += pout
        if ctx.needs_input_grad[0]:
            if stride == 1 and cout % 64 == 0 and cin % 8 == 0:
                # dx = conv(dy, rot180(w) with in/out channels swapped), padding R-1-pad
                w_t = w.flip(2, 3).transpose(0, 1).contiguous(memory_format=torch.channels_last)
                dx2d, _, _ = _conv_native(nhwc_2d(dy_cl), w_t, n, dy.shape[2], dy.shape[3], cout, cin, r, s, 1,
                                          r - 1 - pad, None)
                dx = from_2d(dx2d, n, h, wd)
            elif stride == 2 and r == 3 and s == 3 and pad == 1 and h % 2 == 0 and wd % 2 == 0 and cout % 64 == 0:
                dx = _dgrad_stride2(dy_cl, w, n, h, wd, cin, cout)
            elif pad <= min(r, s) - 1 and cout % 64 == 0 and cin % 8 == 0:
                # Any other stride / size: the gradient is spread out with (stride - 1) zeros between its pixels
                # (plus the rows and columns at the far edge that no window reached) and then goes through the
                # stride-1 form above.  stride^2 times the multiply-adds of a dedicated kernel, but on this
                # package's tensor-core path for every geometry.
                ho, wo = dy_cl.shape[2], dy_cl.shape[3]
                eh, ew = (h + 2 * pad - r) % stride, (wd + 2 * pad - s) % stride
                spread = torch.zeros((n, cout, (ho - 1) * stride + 1 + eh, (wo - 1) * stride + 1 + ew), dtype=dy_cl.dtype,
                                     device=dy_cl.device).contiguous(memory_format=torch.channels_last)
                spread[:, :, :(ho - 1) * stride + 1:stride, :(wo - 1) * stride + 1:stride] = dy_cl
                w_t = w.flip(2, 3).transpose(0, 1).contiguous(memory_format=torch.channels_last)
                dx2d, _, _ = _conv_native(nhwc_2d(spread), w_t, n, spread.shape[2], spread.shape[3], cout, cin, r, s, 1,
                                          r - 1 - pad, None)
                dx = from_2d(dx2d, n, h, wd)
            else:
                dx = torch.nn.grad.conv2d_input((n, cin, h, wd), w, dy_cl, stride=stride, padding=pad)
        if ctx.needs_input_grad[1]:
            from .gemm import error_flag
            cin_w, cin = cin, cin_x            # the weight gradient is taken against the padded input
            dw32 = zeros_f32((cout, r, s, cin), x.device)                               # [Cout][R][S][Cin]
            rc = -100
            if stride == 1:      # shared input boxes, taps as shifted views (returns -100 outside its range)
                rc = _lib().esgd_conv2d_wgrad_halo(nhwc_2d(x).data_ptr(), nhwc_2d(dy_cl).data_ptr(),
                                                   dw32.data_ptr(), n, h, wd, cin, cout, r, s, pad,
                                                   error_flag(x.device).data_ptr(), _stream(x))
                if rc != -100:
                    _ck(rc, "conv2d weight gradient (shared boxes)")
            if rc == -100:
                _ck(_lib().esgd_conv2d_wgrad(nhwc_2d(x).data_ptr(), nhwc_2d(dy_cl).data_ptr(), dw32.data_ptr(), n, h,
                                             wd, cin, cout, r, s, stride, pad, error_flag(x.device).data_ptr(),
                                             _stream(x)), "conv2d weight gradient")
            if pout or cin_w != cin:
                dw32 = dw32[:cout - pout, :, :, :cin_w]
            dw = dw32.to(w.dtype).permute(0, 3, 1, 2)
        return dx, dw, None, None, None


# Narrow convolutions on the tensor-core path by channel padding (ESGD_SMALL_CHANNELS=library keeps them on
# PyTorch's convolution instead).
_SMALL_CHANNELS_NATIVE = os.environ.get("ESGD_SMALL_CHANNELS", "native") != "library"


def _pad_channels(x: torch.Tensor, extra: int) -> torch.Tensor:
    if extra == 0:
        return x
    return F.pad(x, (0, 0, 0, 0, 0, extra)).contiguous(memory_format=torch.channels_last)


class _Subsample2(torch.autograd.Function):
    """x[:, :, ::2, ::2] for NHWC tensors, with a one-pass scatter as its gradient."""

    @staticmethod
    def forward(ctx, x):
        n, c, h, w = x.shape
        x2d = nhwc_2d(x)
        oh, ow = (h + 1) // 2, (w + 1) // 2
        y2d = torch.empty(n * oh * ow, c, dtype=x.dtype, device=x.device)
        _ck(_lib().esgd_subsample2_fwd(x2d.data_ptr(), y2d.data_ptr(), n, h, w, c, _stream(x)), "subsample")
        ctx.dims = (n, c, h, w)
        return from_2d(y2d, n, oh, ow)

    @staticmethod
    def backward(ctx, dy):
        n, c, h, w = ctx.dims
        dy2d = nhwc_2d(dy)
        dx2d = torch.empty(n * h * w, c, dtype=dy.dtype, device=dy.device)
        _ck(_lib().esgd_subsample2_bwd(dy2d.data_ptr(), dx2d.data_ptr(), n, h, w, c, _stream(dy)), "subsample backward")
        return from_2d(dx2d, n, h, w)


def conv2d(x: torch.Tensor, w: torch.Tensor, stride: int = 1, padding: int = 0, want_stats: bool = False,
           tap_input: bool = False):
    """NHWC convolution; returns ``(y, stats)`` (``stats`` is None unless produced by the kernel epilogue).

    1x1 kernels run as tcgen05 GEMMs (a strided 1x1 first gathers the kept pixels).  With ``tap_input`` a
    third value is returned: the tensor a residual block should feed its shortcut from (the input itself, or
    for the fused 1x1 path an alias whose gradient is added inside the data-gradient GEMM).
    """
    if tap_input:
        k1 = w.shape[2] == 1 and stride == 1 and native(x) and x.shape[1] % 8 == 0 and w.shape[0] % 8 == 0
        if k1 and x.requires_grad and torch.is_grad_enabled():
            out = conv1x1(x, w, want_stats, tap_input=True)
            return (out[0], out[1], out[2]) if want_stats else (out[0], None, out[1])
        y, st = conv2d(x, w, stride, padding, want_stats)
        return y, st, x
    k = w.shape[2]
    if k == 1 and native(x) and x.shape[1] % 8 == 0 and w.shape[0] % 8 == 0:
        if stride == 2:
            x = _Subsample2.apply(x)
        elif stride > 1:
            x = x[:, :, ::stride, ::stride].contiguous(memory_format=torch.channels_last)
        out = conv1x1(x, w, want_stats)
        return out if want_stats else (out, None)
    if k > 1 and native(x) and x.shape[1] <= 4 and w.shape[0] % 8 == 0 and not x.requires_grad:
        out = _StemConv.apply(x, w, stride, padding, want_stats)
        return out if want_stats else (out, None)
    if k > 1 and native(x) and x.shape[1] % 64 == 0 and w.shape[0] % 8 == 0 and stride in (1, 2):
        out = _ConvKxK.apply(x, w, stride, padding, want_stats)
        return out if want_stats else (out, None)
    if k > 1 and native(x) and x.shape[1] % 8 == 0 and w.shape[0] % 8 == 0 and stride in (1, 2) and \
            _SMALL_CHANNELS_NATIVE:
        # narrow layers (the 16- and 32-channel stages of the CIFAR ResNets): channel-padded inside the operator
        out = _ConvKxK.apply(x, w, stride, padding, want_stats)
        return out if want_stats else (out, None)
    return F.conv2d(x, w, None, stride, padding), None


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b):
        ctx.save_for_backward(x, w)
        ctx.has_bias = b is not None
        return gemm(x, w, bias=b.float() if b is not None else None, out_dtype=torch.float32)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy16 = dy.to(torch.bfloat16).contiguous()
        dx = gemm(dy16, w, b_kmajor=False) if ctx.needs_input_grad[0] else None
        dw = gemm(dy16, x, a_kmajor=False, b_kmajor=False, out_dtype=torch.float32).to(w.dtype) \
            if ctx.needs_input_grad[1] else None
        db = dy.sum(0).to(w.dtype) if ctx.has_bias and ctx.needs_input_grad[2] else None
        return dx, dw, db


def linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Dense layer; fp32 logits out of bf16 operands on the native path."""
    if native(x) and x.shape[1] % 8 == 0 and w.shape[0] % 8 == 0:
        return _Linear.apply(x.contiguous(), w, b)
    if native(x) and x.shape[1] % 8 == 0 and _SMALL_CHANNELS_NATIVE:
        # a class count that is not a multiple of 8 (10 CIFAR classes, 101 video classes): zero rows are added
        # to the weight so that the tensor-core GEMM can take it, and cut off the logits again
        extra = (-w.shape[0]) % 8
        wp = F.pad(w, (0, 0, 0, extra))
        bp = F.pad(b, (0, extra)) if b is not None else None
        return _Linear.apply(x.contiguous(), wp, bp)[:, :w.shape[0]]
    return F.linear(x, w, b)


# --------------------------------------------------------------------------- batch norm (+ residual) (+ ReLU)
class _BnAct(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, gamma, beta, residual, running_mean, running_var, momentum, relu, stats):
        n, c, h, w = y.shape
        lib = _lib()
        y2d = nhwc_2d(y)
        m = y2d.shape[0]
        s = _stream(y)
        if stats is None:
            stats = torch.zeros(2, c, dtype=torch.float32, device=y.device)
            _ck(lib.esgd_bn_stats(y2d.data_ptr(), m, c, stats[0].data_ptr(), stats[1].data_ptr(), s), "bn_stats")
        aux = torch.empty(4, c, dtype=torch.float32, device=y.device)  # mean, invstd, scale, shift
        _ck(lib.esgd_bn_finalize(stats[0].data_ptr(), stats[1].data_ptr(), gamma.data_ptr(), beta.data_ptr(),
                                 _ptr(running_mean), _ptr(running_var), aux[0].data_ptr(), aux[1].data_ptr(),
                                 aux[2].data_ptr(), aux[3].data_ptr(), c, m, momentum, BN_EPS, s), "bn_finalize")
        r2d = nhwc_2d(residual) if residual is not None else None
        z2d = torch.empty_like(y2d)
        _ck(lib.esgd_bn_apply(y2d.data_ptr(), _ptr(r2d), z2d.data_ptr(), aux[2].data_ptr(), aux[3].data_ptr(), m, c,
                              int(relu), s), "bn_apply")
        ctx.save_for_backward(y2d, z2d, gamma, aux)
        ctx.cfg = (n, h, w, c, relu, residual is not None)
        return from_2d(z2d, n, h, w)

    @staticmethod
    def backward(ctx, dz):
        y2d, z2d, gamma, aux = ctx.saved_tensors
        n, h, w, c, relu, has_res = ctx.cfg
        lib = _lib()
        dz2d = nhwc_2d(dz)
        m = y2d.shape[0]
        s = _stream(dz)
        red = torch.zeros(2, c, dtype=torch.float32, device=dz.device)  # dbeta, dgamma
        # ReLU mask: from the saved output when a residual was added, else recomputed from y (z is not read)
        mode = 0 if not relu else (1 if has_res else 2)
        _ck(lib.esgd_bn_bwd_reduce(dz2d.data_ptr(), z2d.data_ptr(), y2d.data_ptr(), aux[0].data_ptr(),
                                   aux[1].data_ptr(), aux[2].data_ptr(), aux[3].data_ptr(), m, c, mode,
                                   red[0].data_ptr(), red[1].data_ptr(), s), "bn_bwd_reduce")
        dy2d = torch.empty_like(y2d)
        dres2d = torch.empty_like(y2d) if has_res else None
        _ck(lib.esgd_bn_bwd_apply(dz2d.data_ptr(), z2d.data_ptr(), y2d.data_ptr(), aux[0].data_ptr(),
                                  aux[1].data_ptr(), gamma.data_ptr(), red[0].data_ptr(), red[1].data_ptr(),
                                  aux[2].data_ptr(), aux[3].data_ptr(), dy2d.data_ptr(), _ptr(dres2d), m, c, mode,
                                  s), "bn_bwd_apply")
        dres = from_2d(dres2d, n, h, w) if has_res else None
        return from_2d(dy2d, n, h, w), red[1].to(gamma.dtype), red[0].to(gamma.dtype), dres, None, None, None, None, None


def bn_act(y: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, running_mean: Optional[torch.Tensor],
           running_var: Optional[torch.Tensor], momentum: float = 0.003, relu: bool = True,
           residual: Optional[torch.Tensor] = None, stats: Optional[torch.Tensor] = None,
           training: bool = True) -> torch.Tensor:
    """z = act(batch_norm(y) [+ residual]) with batch statistics (training) in fused kernels."""
    if native(y) and training and y.shape[1] % 8 == 0 and gamma.dtype == torch.float32:
        return _BnAct.apply(y, gamma, beta, residual, running_mean, running_var, momentum, relu, stats)
    z = F.batch_norm(y, running_mean, running_var, gamma, beta, training, momentum, BN_EPS)
    if residual is not None:
        z = z + residual
    return F.relu(z) if relu else z


# --------------------------------------------------------------------------- softmax cross-entropy
class _SoftmaxCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, labels):
        lib = _lib()
        b, c = logits.shape
        logits = logits.contiguous()
        loss = torch.zeros(1, dtype=torch.float32, device=logits.device)
        dlogits = torch.empty_like(logits)
        _ck(lib.esgd_softmax_ce(logits.data_ptr(), int(logits.dtype == torch.bfloat16), labels.data_ptr(), b, c,
                                logits.stride(0), 1.0 / b, loss.data_ptr(), None, dlogits.data_ptr(),
                                _stream(logits)), "softmax_ce")
        ctx.save_for_backward(dlogits)
        return loss[0]

    @staticmethod
    def backward(ctx, g):
        (dlogits,) = ctx.saved_tensors
        return dlogits * g, None


def softmax_cross_entropy(logits: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    """Mean sparse softmax cross-entropy; forward and gradient come out of one kernel."""
    if logits.is_cuda and logits.dtype in (torch.float32, torch.bfloat16) and labels.dtype == torch.int64 \
            and not _reference_only:
        return _SoftmaxCE.apply(logits, labels)
    return F.cross_entropy(logits.float(), labels)


# --------------------------------------------------------------------------- pooling
class _MaxPool(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        n, c, h, w = x.shape
        x2d = nhwc_2d(x)
        oh, ow = (h + 1) // 2, (w + 1) // 2
        y2d = torch.empty(n * oh * ow, c, dtype=x.dtype, device=x.device)
        idx = torch.empty(n * oh * ow, c, dtype=torch.uint8, device=x.device)
        _ck(_lib().esgd_maxpool3x3s2_fwd(x2d.data_ptr(), y2d.data_ptr(), idx.data_ptr(), n, h, w, c, _stream(x)),
            "maxpool")
        ctx.save_for_backward(idx)
        ctx.dims = (n, c, h, w, oh, ow)
        return from_2d(y2d, n, oh, ow)

    @staticmethod
    def backward(ctx, dy):
        (idx,) = ctx.saved_tensors
        n, c, h, w, oh, ow = ctx.dims
        dy2d = nhwc_2d(dy)
        dx2d = torch.empty(n * h * w, c, dtype=dy.dtype, device=dy.device)
        _ck(_lib().esgd_maxpool3x3s2_bwd(idx.data_ptr(), dy2d.data_ptr(), dx2d.data_ptr(), n, h, w, c, _stream(dy)),
            "maxpool backward")
        return from_2d(dx2d, n, h, w)


def max_pool_3x3_s2(x: torch.Tensor) -> torch.Tensor:
    if native(x) and x.shape[1] % 8 == 0:
        return _MaxPool.apply(x)
    return F.max_pool2d(x, 3, 2, 1)


class _AvgPool(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        n, c, h, w = x.shape
        x2d = nhwc_2d(x)
        y = torch.empty(n, c, dtype=x.dtype, device=x.device)
        _ck(_lib().esgd_avgpool_fwd(x2d.data_ptr(), y.data_ptr(), n, h * w, c, _stream(x)), "avgpool")
        ctx.dims = (n, c, h, w)
        return y

    @staticmethod
    def backward(ctx, dy):
        n, c, h, w = ctx.dims
        dy = dy.contiguous()
        dx2d = torch.empty(n * h * w, c, dtype=dy.dtype, device=dy.device)
        _ck(_lib().esgd_avgpool_bwd(dy.data_ptr(), dx2d.data_ptr(), n, h * w, c, _stream(dy)), "avgpool backward")
        return from_2d(dx2d, n, h, w)


def global_avg_pool(x: torch.Tensor) -> torch.Tensor:
    """[N, C, H, W] -> [N, C] mean over H, W."""
    if native(x) and x.shape[1] % 8 == 0:
        return _AvgPool.apply(x)
    return torch.flatten(F.adaptive_avg_pool2d(x, 1), 1)
