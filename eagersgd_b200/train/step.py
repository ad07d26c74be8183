"""One training step of an image classifier: the call a user of the framework makes.

``TrainStep`` prepares the model for B200 (NHWC activations, bf16 weights for
convolutions and dense layers with fp32 master copies, fp32 batch-norm), wraps
momentum SGD in one of the eager-SGD optimizers and exposes

* ``run_device(x, y)``: forward, backward, partial allreduce + fused update,
  inputs already on the GPU, no host synchronisation;
* ``run_host(x_pinned, y_pinned)``: the same, end to end — host-to-device copy of
  the batch from pinned memory first, device-to-host read of the loss last.

It stands where the reference's ``resnet_model_fn`` builds loss, optimizer wrap and
train op (official/resnet/resnet_run_loop_solo_imagenet_300.py:220-456).
"""
from __future__ import annotations

from typing import Optional

import contextlib

import torch
import torch.nn as nn

from ..optim.eager import MajorityAllreduceOptimizer, SoloAllreduceOptimizer, SyncAllreduceOptimizer
from ..parallel import _native as N
from ..parallel.group import Group
from ..utils.nvtx import nvtx_range


def prepare_model(model: nn.Module, device: torch.device, compute_dtype=torch.bfloat16) -> nn.Module:
    """NHWC, low-precision conv/dense weights, fp32 normalisation layers."""
    model = model.to(device)
    if device.type == "cuda":
        model = model.to(memory_format=torch.channels_last)
        if hasattr(model, "compute_dtype_"):        # models with their own parameter containers
            model.compute_dtype_(compute_dtype)
        for m in model.modules():
            if isinstance(m, (nn.Conv2d, nn.Linear, nn.LSTM)):
                m.to(compute_dtype)
    return model


class TrainStep:
    def __init__(self, model: nn.Module, group: Group, impl: str = "ours", mode: str = "solo", limiter: int = 32,
                 bucket_mb: float = 25.0, lr: float = 0.01, momentum: float = 0.9, weight_decay: float = 1e-4,
                 compute_dtype=torch.bfloat16, loss_fn=None, inner_optimizer=None, loss_scale: float = 1.0,
                 accumulate: bool = False, decay_norm_params: bool = True):
        """``decay_norm_params=False`` keeps weight decay off the scale and shift of the normalisation layers, as the
        reference's ImageNet objective does (its L2 term skips every variable with 'batch_normalization' in its name,
        resnet_run_loop_solo_imagenet_300.py:328-339; its CIFAR-10 objective includes them, cifar10_main.py:244-250):
        the optimizer then has two parameter groups."""
        self.group, self.impl, self.device = group, impl, group.device
        self.compute_dtype = compute_dtype if self.device.type == "cuda" else torch.float32
        self.loss_scale = float(loss_scale)
        from ..ops.functional import softmax_cross_entropy
        self.loss_fn = loss_fn or softmax_cross_entropy
        if impl == "ddp":
            self.model = model.to(self.device)
            if self.device.type == "cuda":
                self.model = self.model.to(memory_format=torch.channels_last)
            self.net = self.model
            if group.world > 1:
                from torch.nn.parallel import DistributedDataParallel as DDP
                self.net = DDP(self.model, device_ids=[self.device.index] if self.device.type == "cuda" else None,
                               bucket_cap_mb=bucket_mb, gradient_as_bucket_view=True)
            self.opt = torch.optim.SGD(self._param_groups(self.model, weight_decay, decay_norm_params), lr=lr,
                                       momentum=momentum, weight_decay=weight_decay)
            self.autocast = self.device.type == "cuda"
        else:
            self.model = prepare_model(model, self.device, self.compute_dtype)
            self.net = self.model
            if inner_optimizer is not None:      # any torch optimizer can be wrapped (LARS, Adam, ...)
                inner = inner_optimizer(self.model.parameters(), lr=lr)
            else:
                inner = torch.optim.SGD(self._param_groups(self.model, weight_decay, decay_norm_params), lr=lr,
                                        momentum=momentum, weight_decay=weight_decay)
            cls = {"solo": SoloAllreduceOptimizer, "majority": MajorityAllreduceOptimizer,
                   "sync": SyncAllreduceOptimizer}[mode]
            kw = dict(bucket_mb=bucket_mb, accumulate=accumulate)
            if mode != "sync":
                kw["limiter"] = limiter
            self.opt = cls(inner, group, **kw)
            self.opt.grad_scale = 1.0 / self.loss_scale   # static loss scaling is undone inside the update
            self.autocast = False
        n_params = sum(p.numel() for p in self.net.parameters())
        self._arena_numel = n_params + 64 * (len(list(self.net.parameters())) + 8) + (1 << 20)
        self._xbuf = self._ybuf = None
        self._graph = None
        self.graph_kernel_launches = 0

    @staticmethod
    def _param_groups(model: nn.Module, weight_decay: float, decay_norm_params: bool):
        """All parameters in one group, or — to keep weight decay off the normalisation layers — two."""
        if decay_norm_params or not weight_decay:
            return list(model.parameters())
        norm = {id(p) for m in model.modules() if isinstance(m, nn.modules.batchnorm._BatchNorm) for p in m.parameters(recurse=False)}
        decayed = [p for p in model.parameters() if id(p) not in norm]
        plain = [p for p in model.parameters() if id(p) in norm]
        if not plain:
            return decayed
        return [{"params": decayed}, {"params": plain, "weight_decay": 0.0}]

    def capture(self, x: torch.Tensor, y: torch.Tensor, warmup: int = 2) -> None:
        """Capture the whole step (forward, backward, bucketed partial allreduce with the
        fused update on its side stream) into one CUDA graph: a replay costs one launch.
        ``warmup`` real training steps run first; every rank must call this the same way."""
        assert self.device.type == "cuda" and self.impl != "ddp"
        if not getattr(self.opt, "fused", False):
            # A wrapped optimizer (LARS, Adam, ...) takes its learning rate as a host value at every step and is
            # skipped on the host when the rank applied nothing: neither survives being recorded once.
            raise NotImplementedError("only the fused momentum-SGD path can be captured in a CUDA graph; "
                                      "run a wrapped optimizer without capture")
        self._gx, self._gy = x.clone(), y.clone()
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            for _ in range(warmup):
                self._step(self._gx, self._gy)
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        n0 = N.launch_count()
        with torch.cuda.graph(graph):
            self._gloss = self._step(self._gx, self._gy)
        self.graph_kernel_launches = N.launch_count() - n0   # kernels of this package inside one replay
        self._graph = graph

    def run_device(self, x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        if self._graph is not None:
            if x.data_ptr() != self._gx.data_ptr():
                self._gx.copy_(x, non_blocking=True)
                self._gy.copy_(y, non_blocking=True)
            self.opt.sync_hyper()
            self._graph.replay()
            return self._gloss
        return self._step(x, y)

    def _step(self, x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        self.opt.zero_grad()
        if self.impl == "ddp":
            # the baseline arm: PyTorch's own operators (cuDNN / cuBLAS) under bf16 autocast
            from ..ops.functional import reference_ops
            with reference_ops():
                with torch.autocast("cuda", dtype=torch.bfloat16, enabled=self.autocast):
                    logits = self.net(x.float() if self.device.type != "cuda" else x)
                loss = torch.nn.functional.cross_entropy(logits.float(), y)
            loss.backward()
            self.opt.step()
            return loss.detach()
        from ..ops.functional import zero_arena
        # every operator's zeroed fp32 scratch (statistics, weight-gradient accumulators) comes out of one
        # buffer cleared by a single memset per step
        with zero_arena(self.device, self._arena_numel) if self.device.type == "cuda" else contextlib.nullcontext():
            with nvtx_range("forward"):
                logits = self.net(x if x.dtype == self.compute_dtype or not x.is_floating_point()
                                  else x.to(self.compute_dtype))
                loss = self.loss_fn(logits if logits.dtype == torch.float32 else logits.float(), y)
            with nvtx_range("backward"):
                (loss * self.loss_scale if self.loss_scale != 1.0 else loss).backward()
        with nvtx_range("optimizer"):
            self.opt.step()
        return loss.detach()

    def run_host(self, x_host: torch.Tensor, y_host: torch.Tensor) -> float:
        """End to end: pinned host batch in, python float loss out."""
        if self._graph is not None:
            self._xbuf, self._ybuf = self._gx, self._gy   # copy straight into the graph's input buffers
        elif self._xbuf is None or self._xbuf.shape != x_host.shape:
            self._xbuf = torch.empty_like(x_host, device=self.device)
            self._ybuf = torch.empty_like(y_host, device=self.device)
        self._xbuf.copy_(x_host, non_blocking=True)
        self._ybuf.copy_(y_host, non_blocking=True)
        return float(self.run_device(self._xbuf, self._ybuf).item())

    def run_host_stream(self, batches, before_step=None):
        """End to end over a stream of pinned host batches, pipelined: yields every step's loss as a python float, in
        order.  The host-to-device copy of batch k+1 runs on a copy stream while step k computes (two staging buffers
        on the device), and the loss of step k is read back (asynchronous copy into pinned memory) only after step
        k+1 has been launched, so neither transfer leaves the GPU idle.  ``before_step(k)`` is called right before
        step k is launched (the benchmark injects its delays there).  On a CPU device this is ``run_host`` in a loop."""
        if self.device.type != "cuda":
            for k, (xh, yh) in enumerate(batches):
                if before_step is not None:
                    before_step(k)
                yield self.run_host(xh, yh)
            return
        dev = self.device
        main = torch.cuda.current_stream(dev)
        if getattr(self, "_copy_stream", None) is None:
            self._copy_stream = torch.cuda.Stream(device=dev)
            self._stage = [None, None]
            self._loss_pin = [torch.zeros(1, dtype=torch.float32).pin_memory() for _ in range(2)]
        copy = self._copy_stream
        h2d_done = [torch.cuda.Event() for _ in range(2)]
        stage_free = [torch.cuda.Event() for _ in range(2)]
        loss_done = [torch.cuda.Event() for _ in range(2)]

        def prefetch(k, xh, yh):
            b = k % 2
            st = self._stage[b]
            if st is None or st[0].shape != xh.shape or st[0].dtype != xh.dtype or st[1].shape != yh.shape:
                # From the copy stream's pool, and marked as used by the compute stream: memory that the compute
                # stream has freed but whose kernels are still queued must not be written by an early copy, and a
                # staging buffer dropped here must not be handed out again before the step that reads it is done.
                with torch.cuda.stream(copy):
                    st = self._stage[b] = (torch.empty_like(xh, device=dev), torch.empty_like(yh, device=dev))
                for t in st:
                    t.record_stream(main)
            if k >= 2:
                copy.wait_event(stage_free[b])           # the step that read this buffer two batches ago is past it
            else:
                copy.wait_stream(main)
            with torch.cuda.stream(copy):
                st[0].copy_(xh, non_blocking=True)
                st[1].copy_(yh, non_blocking=True)
                h2d_done[b].record(copy)

        it = iter(batches)
        nxt = next(it, None)
        if nxt is None:
            return
        prefetch(0, *nxt)
        k = 0
        while nxt is not None:
            b = k % 2
            main.wait_event(h2d_done[b])
            x, y = self._stage[b]
            if self._graph is not None:                  # the graph reads fixed buffers: one device copy into them
                self._gx.copy_(x, non_blocking=True)
                self._gy.copy_(y, non_blocking=True)
                stage_free[b].record(main)
                x, y = self._gx, self._gy
            nxt = next(it, None)
            if nxt is not None and self._graph is not None:
                prefetch(k + 1, *nxt)
            if before_step is not None:
                before_step(k)
            loss = self.run_device(x, y)
            if self._graph is None:
                stage_free[b].record(main)
                if nxt is not None:
                    prefetch(k + 1, *nxt)
            self._loss_pin[b].copy_(loss.detach().reshape(1).float(), non_blocking=True)
            loss_done[b].record(main)
            if k > 0:
                loss_done[1 - b].synchronize()
                yield float(self._loss_pin[1 - b][0])
            k += 1
        loss_done[(k - 1) % 2].synchronize()
        yield float(self._loss_pin[(k - 1) % 2][0])

    def set_lr(self, lr: float) -> None:
        for g in self.opt.param_groups:
            g["lr"] = lr

    def inject_delay(self, seconds: float) -> None:
        """Seeded load imbalance: hold this rank's compute stream (GPU) or sleep (CPU)."""
        if self.device.type == "cuda":
            N.check_cuda(N.cuda().esgd_spin(int(seconds * 1e9), torch.cuda.current_stream(self.device).cuda_stream),
                         "delay injection")
        else:
            import time
            time.sleep(seconds)

    def stats(self) -> Optional[dict]:
        return self.opt.stats() if hasattr(self.opt, "stats") else None

    def close(self) -> None:
        if hasattr(self.opt, "close"):
            self.opt.close()
