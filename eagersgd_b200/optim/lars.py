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
