"""LARS (layer-wise adaptive rate scaling) and its polynomial learning-rate schedule.

Trust ratio ``eeta * ||w|| / (||g|| + wd * ||w|| + eps)`` per tensor, momentum on the scaled
gradient, no adaptation for excluded (bias / batch-norm) tensors — the reference's
LARSOptimizer (official/utils/lars_optimizer.py:101-115) and poly schedule
(official/resnet/lars_util.py:30-80).  The norms of all tensors are taken with two
multi-tensor reductions per step.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch


class LARS(torch.optim.Optimizer):
    def __init__(self, params, lr: float = 0.1, momentum: float = 0.9, weight_decay: float = 1e-4,
                 eeta: float = 0.001, epsilon: float = 0.0, skip: Optional[Callable[[torch.Tensor], bool]] = None):
        super().__init__(params, dict(lr=lr, momentum=momentum, weight_decay=weight_decay, eeta=eeta,
                                      epsilon=epsilon))
        # tensors with one dimension (biases, batch-norm scale / shift) are not adapted
        self.skip = skip or (lambda p: p.dim() <= 1)

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for g in self.param_groups:
            ps = [p for p in g["params"] if p.grad is not None]
            if not ps:
                continue
            w_norms = torch._foreach_norm([p.float() for p in ps])
            g_norms = torch._foreach_norm([p.grad.float() for p in ps])
            for p, wn, gn in zip(ps, w_norms, g_norms):
                grad = p.grad.float()
                lr = g["lr"]
                if not self.skip(p):
                    trust = torch.where((wn > 0) & (gn > 0),
                                        g["eeta"] * wn / (gn + g["weight_decay"] * wn + g["epsilon"]),
                                        torch.ones_like(wn))
                    grad = (grad + g["weight_decay"] * p.float()) * trust
                buf = self.state[p].get("momentum_buffer")
                if buf is None:
                    buf = self.state[p]["momentum_buffer"] = torch.zeros_like(p, dtype=torch.float32)
                buf.mul_(g["momentum"]).add_(grad, alpha=lr)
                p.add_(-buf.to(p.dtype))
        return loss


class FusedLARS:
    """LARS on the GPU in two kernel launches per step (per-tensor norms, then the update with fp32 master
    weights, momentum and a bf16 copy for the model), whatever the number of tensors.  Same rule as ``LARS``;
    parameters live in flat buffers like ``FusedSGD``'s.  ``step()`` never synchronises with the host."""

    def __init__(self, params, lr: float = 0.1, momentum: float = 0.9, weight_decay: float = 1e-4,
                 eeta: float = 0.001, epsilon: float = 0.0, skip: Optional[Callable[[torch.Tensor], bool]] = None):
        import ctypes as C

        import numpy as np

        from ..parallel import _native as N
        self._N, self._C = N, C
        self.params = [p for p in params if p.requires_grad]
        dev, dt = self.params[0].device, self.params[0].dtype
        if dev.type != "cuda" or any(p.dtype != dt for p in self.params) or dt not in (torch.float32, torch.bfloat16):
            raise ValueError("FusedLARS needs CUDA parameters of one dtype, float32 or bfloat16")
        self.lr, self.momentum, self.weight_decay, self.eeta, self.epsilon = lr, momentum, weight_decay, eeta, epsilon
        self.grad_scale = 1.0
        skip = skip or (lambda p: p.dim() <= 1)
        lib = N.cuda()
        lib.esgd_lars_step.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_float,
                                       C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_float, C.c_float, C.c_float,
                                       C.c_float, C.c_void_p]
        chunk = int(lib.esgd_lars_chunk_elems())
        assert int(lib.esgd_lars_chunk_bytes()) == 16
        self.offsets, n, recs = [], 0, []
        for t, p in enumerate(self.params):
            self.offsets.append(n)
            padded = (p.numel() + 63) // 64 * 64
            for s0 in range(0, padded, chunk):
                recs.append((n + s0, min(chunk, padded - s0), (-1 - t) if skip(p) else t))
            n += padded
        self.count = n
        rec = np.zeros(len(recs), dtype=np.dtype([("start", "<i8"), ("len", "<i4"), ("tensor", "<i4")]))
        for i, r in enumerate(recs):
            rec[i] = r
        self._chunks = torch.from_numpy(rec.view(np.uint8).copy()).to(dev)
        self._num_chunks = len(recs)
        self._sq = torch.zeros(2 * len(self.params), dtype=torch.float32, device=dev)
        self.w32 = torch.zeros(n, dtype=torch.float32, device=dev)
        self.mom = torch.zeros(n, dtype=torch.float32, device=dev)
        self.w16 = torch.zeros(n, dtype=dt, device=dev) if dt != torch.float32 else None
        self.grad = torch.zeros(n, dtype=dt, device=dev)
        for p, off in zip(self.params, self.offsets):
            k = p.numel()
            self.w32[off:off + k].copy_(p.detach().reshape(-1).float())
            store = self.w16 if self.w16 is not None else self.w32
            if self.w16 is not None:
                store[off:off + k].copy_(p.detach().reshape(-1))
            p.data = store[off:off + k].view(p.shape)
            p.grad = self.grad[off:off + k].view(p.shape)

    def zero_grad(self, set_to_none: bool = False):
        self.grad.zero_()

    def step(self):
        s = torch.cuda.current_stream(self.w32.device).cuda_stream
        self._N.check_cuda(self._N.cuda().esgd_lars_step(
            self._chunks.data_ptr(), self._num_chunks, len(self.params), self._sq.data_ptr(), self.grad.data_ptr(),
            int(self.grad.dtype == torch.bfloat16), self.grad_scale, self.w32.data_ptr(), self.mom.data_ptr(),
            self.w16.data_ptr() if self.w16 is not None else None, self.lr, self.momentum, self.weight_decay,
            self.eeta, self.epsilon, s), "fused LARS")


def poly_rate_schedule(current_epoch: float, poly_rate: float = 0.0, batch_size: int = 8192,
                       train_epochs: int = 90, warmup_epochs: Optional[float] = None) -> float:
    """Linear warm-up then (1 - t)^2 decay; the plateau rate follows the batch size when
    ``poly_rate`` is 0 (lars_util.py:30-80)."""
    if poly_rate == 0.0:
        poly_rate = 5.0 if batch_size < 8192 else (10.0 if batch_size < 16384 else (25.0 if batch_size < 32768 else 32.0))
    if warmup_epochs is None:
        warmup_epochs = 5 if batch_size < 16384 else (14 if batch_size < 32768 else 27)  # batch-size dependent
    if current_epoch < warmup_epochs:
        return poly_rate * current_epoch / warmup_epochs
    t = (current_epoch - warmup_epochs) / max(train_epochs - warmup_epochs, 1e-9)
    return poly_rate * max(0.0, 1.0 - t) ** 2
