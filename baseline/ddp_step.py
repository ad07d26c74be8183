"""The synchronous PyTorch baseline step: ``DistributedDataParallel`` over NCCL, bf16 autocast, channels_last,
cuDNN / cuBLAS kernels, fused momentum SGD.  Same interface as ``eagersgd_b200.train.step.TrainStep``
(``run_device`` / ``run_host`` / ``inject_delay`` / ``capture`` / ``close``) so that ``bench.py`` can time it the same
way.  On one GPU the whole step is captured in a CUDA graph (nothing to synchronise with); on several GPUs
it runs the way PyTorch users run it, eagerly with DDP's bucketed allreduce overlapping backward.
"""
from __future__ import annotations

import torch
import torch.nn as nn


class DDPStep:
    def __init__(self, model: nn.Module, group, bucket_mb: float = 25.0, lr: float = 0.01, momentum: float = 0.9,
                 weight_decay: float = 1e-4, channels_last: bool = True):
        self.group, self.device = group, group.device
        self.model = model.to(self.device)
        if channels_last:
            self.model = self.model.to(memory_format=torch.channels_last)
        self.net = self.model
        if group.world > 1:
            from torch.nn.parallel import DistributedDataParallel as DDP
            self.net = DDP(self.model, device_ids=[self.device.index], bucket_cap_mb=bucket_mb,
                           gradient_as_bucket_view=True, static_graph=True)
        try:
            self.opt = torch.optim.SGD(self.model.parameters(), lr=lr, momentum=momentum, weight_decay=weight_decay,
                                       fused=True)
        except (TypeError, RuntimeError):
            self.opt = torch.optim.SGD(self.model.parameters(), lr=lr, momentum=momentum, weight_decay=weight_decay)
        self._graph = None
        self._xbuf = self._ybuf = None
        self.graph_kernel_launches = 0

    def _step(self, x, y):
        self.opt.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            logits = self.net(x)
        loss = nn.functional.cross_entropy(logits.float(), y)
        loss.backward()
        self.opt.step()
        return loss.detach()

    def capture(self, x, y, warmup: int = 3):
        if self.group.world > 1:
            return      # eager DDP
        self._gx, self._gy = x.clone(), y.clone()
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            for _ in range(warmup):
                self._step(self._gx, self._gy)
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        self.opt.zero_grad(set_to_none=True)
        with torch.cuda.graph(g):
            self._gloss = self._step(self._gx, self._gy)
        self._graph = g

    def run_device(self, x, y):
        if self._graph is not None:
            if x.data_ptr() != self._gx.data_ptr():
                self._gx.copy_(x, non_blocking=True)
                self._gy.copy_(y, non_blocking=True)
            self._graph.replay()
            return self._gloss
        return self._step(x, y)

    def run_host(self, x_host, y_host) -> float:
        if self._graph is not None:
            self._xbuf, self._ybuf = self._gx, self._gy
        elif self._xbuf is None or self._xbuf.shape != x_host.shape:
            self._xbuf = torch.empty_like(x_host, device=self.device)
            self._ybuf = torch.empty_like(y_host, device=self.device)
        self._xbuf.copy_(x_host, non_blocking=True)
        self._ybuf.copy_(y_host, non_blocking=True)
        return float(self.run_device(self._xbuf, self._ybuf).item())

    def inject_delay(self, seconds: float) -> None:
        """The same injector as the other arms: a bounded spin on this rank's compute stream."""
        from eagersgd_b200.parallel import _native as N
        N.check_cuda(N.cuda().esgd_spin(int(seconds * 1e9), torch.cuda.current_stream(self.device).cuda_stream),
                     "delay injection")

    def stats(self):
        return None

    def close(self):
        self._graph = None
        self.net = self.model = self.opt = None
