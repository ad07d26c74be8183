"""Fused momentum SGD over flat fp32 master weights with a bf16 copy for the model.

One kernel pass per step (weight decay, momentum, update, bf16 write-back): the stand-alone
form of the update the partial-allreduce kernel applies in its epilogue.  Semantics of
``torch.optim.SGD`` (dampening 0); the reference uses TensorFlow's ApplyMomentum
(official/resnet/resnet_run_loop_solo_imagenet_300.py:371-374) and keeps fp32 master variables
under fp16 compute (official/resnet/resnet_model.py:435-474).
"""
from __future__ import annotations

import torch

from ..parallel import _native as N


class FusedSGD:
    def __init__(self, params, lr: float = 0.1, momentum: float = 0.9, weight_decay: float = 0.0,
                 nesterov: bool = False):
        self.params = [p for p in params if p.requires_grad]
        dev, dt = self.params[0].device, self.params[0].dtype
        assert dev.type == "cuda" and all(p.dtype == dt for p in self.params)
        self.lr, self.momentum, self.weight_decay, self.nesterov = lr, momentum, weight_decay, nesterov
        self.offsets, n = [], 0
        for p in self.params:
            self.offsets.append(n)
            n += (p.numel() + 63) // 64 * 64
        self.count = n
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
        N.check_cuda(N.cuda().esgd_fused_sgd(self.grad.data_ptr(), int(self.grad.dtype == torch.bfloat16),
                                             self.w32.data_ptr(), self.mom.data_ptr(),
                                             self.w16.data_ptr() if self.w16 is not None else None, self.count,
                                             self.lr, self.momentum, self.weight_decay, int(self.nesterov), 1.0, s),
                     "fused SGD")
