"""Eager-SGD optimizer wrappers: solo, majority and synchronous partial allreduce.

``SoloAllreduceOptimizer`` / ``MajorityAllreduceOptimizer`` /
``SyncAllreduceOptimizer`` wrap any ``torch.optim.Optimizer`` the way the
reference's ``EagerSGDOptimizer(optimizer, comm_size)`` wraps a TF optimizer
(test-models/.../official/utils/opt_esgd_solo_imagenet_imbalance.py:6-44,
opt_esgd_majority_imagenet_imbalance.py, opt_sgd_mpi.py).  Differences by
design: gradients travel in ~25 MB buckets instead of one blocking collective
per tensor, each bucket is launched on a side stream as soon as backward has
produced it, and on GPUs the reduction is fused with the momentum-SGD update
when the wrapped optimizer is ``torch.optim.SGD``.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import numpy as np
import torch

from ..parallel import _native as N
from ..parallel.group import Group, init as init_group
from ..parallel.nvlink_channel import TWO_SHOT_MIN
from ..utils.nvtx import nvtx_range

_PAD = 64  # elements; keeps every parameter 128-byte aligned inside a bucket


class _Bucket:
    def __init__(self, index: int, group_index: int):
        self.index = index
        self.group_index = group_index
        self.params: List[torch.nn.Parameter] = []
        self.offsets: List[int] = []
        self.count = 0
        self.pending = 0
        self.launched = False
        self.channel = None
        self.grad_flat = None
        self.w32 = self.mom = self.w16 = self.g32 = None
        self.masters = None
        self.hyper = None
        self.hyper_vals = None
        self.self_clearing = False
        self.dirty = True

    def add(self, p):
        self.params.append(p)
        self.offsets.append(self.count)
        self.count += (p.numel() + _PAD - 1) // _PAD * _PAD


def _view_like(flat: torch.Tensor, off: int, p: torch.Tensor) -> torch.Tensor:
    """A view of ``flat`` with the shape *and memory format* of ``p``."""
    n = p.numel()
    seg = flat[off:off + n]
    if p.dim() == 4 and not p.is_contiguous() and p.is_contiguous(memory_format=torch.channels_last):
        o, i, h, w = p.shape
        return seg.view(o, h, w, i).permute(0, 3, 1, 2)
    return seg.view(p.shape)


class EagerOptimizer:
    """Base wrapper.  ``mode`` is 'solo', 'majority' or 'sync'."""

    def __init__(self, optimizer: torch.optim.Optimizer, group: Optional[Group] = None, mode: str = "solo",
                 limiter: int = 32, seed: int = 6545343, bucket_mb: float = 25.0,
                 average: str = "contributors", include_stale: bool = True, fused: Optional[bool] = None,
                 slot_dtype: Optional[torch.dtype] = None, overlap: bool = True, timeout_s: float = 30.0,
                 grace_us: float = 50.0, max_blocks: int = 592, two_shot_min: Optional[int] = TWO_SHOT_MIN,
                 accumulate: bool = False, adaptive_grace: bool = True):
        self.optimizer = optimizer
        self.two_shot_min = two_shot_min   # bucket elements from which a round is reduced in two shots (None: never)
        # fold a gradient that no round picked up into this rank's next publish instead of dropping it
        # (the reference drops it: opt_esgd_solo_imagenet_imbalance.py:311-314 zeroes the send buffer)
        self.accumulate = accumulate
        self.adaptive_grace = adaptive_grace
        self.group = group if group is not None else init_group()
        self.mode, self.limiter, self.seed = mode, limiter, seed
        self.average, self.include_stale = average, include_stale
        self.overlap = overlap
        self.timeout_s, self.grace_us, self.max_blocks = timeout_s, grace_us, max_blocks
        self.steps = 0
        self.grad_scale = 1.0   # multiplies every gradient before the update (1 / loss scale)
        params = [p for g in optimizer.param_groups for p in g["params"] if p.requires_grad]
        if not params:
            raise ValueError("optimizer has no trainable parameters")
        self.device = params[0].device
        self.on_gpu = self.device.type == "cuda"
        if self.on_gpu:
            bad = sorted({str(p.dtype) for p in params if p.dtype not in (torch.float32, torch.bfloat16)})
            if bad:
                raise ValueError("the GPU partial allreduce handles float32 and bfloat16 parameters only (found %s); "
                                 "use bfloat16 for low-precision compute" % ", ".join(bad))
            if slot_dtype not in (None, torch.float32, torch.bfloat16):
                raise ValueError("slot_dtype must be torch.float32 or torch.bfloat16")
        can_fuse = (self.on_gpu and type(optimizer) is torch.optim.SGD and
                    all(g.get("dampening", 0) == 0 and not g.get("maximize", False) for g in optimizer.param_groups))
        self.fused = can_fuse if fused is None else (fused and can_fuse)
        # LARS is the other optimizer the reference wraps (resnet_run_loop_solo_imagenet_300.py:366-374): on
        # GPUs its step runs as two kernels over the buckets' flat buffers instead of a Python loop over tensors
        self.lars = bool(self.on_gpu and type(optimizer).__name__ == "LARS" and not self.fused)
        if slot_dtype is None:
            slot_dtype = torch.bfloat16 if params[0].dtype == torch.bfloat16 else torch.float32
        self.slot_dtype = slot_dtype
        self._build_buckets(bucket_mb)
        self._hooks = []
        if self.on_gpu:
            self._setup_gpu()
            self._install_hooks()
        else:
            self._setup_cpu()

    # ------------------------------------------------------------------ buckets
    def _build_buckets(self, bucket_mb: float):
        esz = 2 if self.slot_dtype == torch.bfloat16 else 4
        cap = max(int(bucket_mb * (1 << 20) / esz), 1)
        self.buckets: List[_Bucket] = []
        for gi, g in enumerate(self.optimizer.param_groups):
            open_by_dtype: Dict[torch.dtype, _Bucket] = {}
            # reverse order: the last layers' gradients are ready first (the reference
            # walks reversed(grads_and_vars) too, opt_esgd_solo_imagenet_imbalance.py:28);
            # one open bucket per dtype, so bf16 weights and fp32 norm parameters do not
            # fragment each other's buckets
            for p in reversed([p for p in g["params"] if p.requires_grad]):
                cur = open_by_dtype.get(p.dtype)
                if cur is None or (cur.count + p.numel() > cap and cur.count > 0):
                    cur = _Bucket(len(self.buckets), gi)
                    self.buckets.append(cur)
                    open_by_dtype[p.dtype] = cur
                cur.add(p)
        self._bucket_of: Dict[int, _Bucket] = {}
        for b in self.buckets:
            b.count = (b.count + 7) // 8 * 8
            for p in b.params:
                self._bucket_of[id(p)] = b

    def _point_grads(self, b: _Bucket):
        for p, off in zip(b.params, b.offsets):
            p.grad = _view_like(b.grad_flat, off, p)

    # ------------------------------------------------------------------ CPU
    def _setup_cpu(self):
        from ..parallel.cpu_channel import CpuChannel, LocalSegments, SharedSegments
        g = self.group
        self._segments = []
        for b in self.buckets:
            dt = b.params[0].dtype
            if dt not in (torch.float32, torch.float64):
                raise ValueError("the CPU backend reduces float32/float64 parameters")
            npdt = np.float32 if dt == torch.float32 else np.float64
            b.grad_flat = torch.zeros(b.count, dtype=dt)
            self._point_grads(b)
            if g.world == 1:
                seg = LocalSegments(1, b.count, npdt)
            else:
                seg = SharedSegments(g.rank, g.world, b.count, npdt, g.exchange)
            self._segments.append(seg)
            b.channel = CpuChannel(seg.bases, g.rank, g.world, b.count, npdt, mode=self.mode, limiter=self.limiter,
                                   seed=self.seed, average=self.average,
                                   include_stale=self.include_stale, timeout_s=self.timeout_s,
                                   grace_us=self.grace_us, accumulate=self.accumulate,
                                   adaptive_grace=self.adaptive_grace)
            b.out_np = np.empty(b.count, dtype=npdt)

    # ------------------------------------------------------------------ GPU
    def _setup_gpu(self):
        from ..parallel.nvlink_channel import HYPER_LEN, NvlinkChannel, create_arenas
        g = self.group
        self.comm_stream = torch.cuda.Stream(device=self.device, priority=-1)
        self._arenas = []
        master_of = {}
        for b in self.buckets:
            dt = b.params[0].dtype
            low = dt != torch.float32
            b.grad_flat = torch.zeros(b.count, dtype=dt, device=self.device)
            b.hyper = torch.zeros(HYPER_LEN, dtype=torch.float32, device=self.device)
            b.masters = None
            if self.fused or low or self.lars:
                # fp32 master weights; the model computes on the bucket's own (low-precision) storage
                b.w32 = torch.zeros(b.count, dtype=torch.float32, device=self.device)
                if low:
                    b.w16 = torch.zeros(b.count, dtype=dt, device=self.device)
                store = b.w16 if low else b.w32
                for p, off in zip(b.params, b.offsets):
                    _view_like(b.w32, off, p).copy_(p.detach().float())
                    v = _view_like(store, off, p)
                    if low:
                        v.copy_(p.detach())
                    p.data = v
            if self.fused:
                b.mom = torch.zeros(b.count, dtype=torch.float32, device=self.device)
                kw = dict(w32=b.w32, mom=b.mom, w16=b.w16, clear_grad=True)
            elif self.lars:
                b.g32 = torch.zeros(b.count, dtype=torch.float32, device=self.device)
                b.mom = torch.zeros(b.count, dtype=torch.float32, device=self.device)
                self._lars_tables(b)
                kw = dict(out=b.g32, clear_grad=True)
            elif low:
                # a wrapped optimizer steps the fp32 masters with the averaged gradient in fp32; the
                # low-precision weights are refreshed from them after every step
                b.g32 = torch.zeros(b.count, dtype=torch.float32, device=self.device)
                b.masters = []
                for p, off in zip(b.params, b.offsets):
                    m = torch.nn.Parameter(_view_like(b.w32, off, p), requires_grad=True)
                    m.grad = _view_like(b.g32, off, p)
                    b.masters.append(m)
                    master_of[id(p)] = m
                kw = dict(out=b.g32, clear_grad=True)
            else:
                kw = dict(out=b.grad_flat)
            b.self_clearing = bool(kw.get("clear_grad", False))
            b.dirty = False
            self._point_grads(b)
            arena, bases = create_arenas(b.count, self.slot_dtype, g.rank, g.world, g.exchange)
            self._arenas.append(arena)
            b.channel = NvlinkChannel(b.count, g.rank, g.world, bases, self.device, b.grad_flat,
                                      slot_dtype=self.slot_dtype, mode=self.mode, limiter=self.limiter,
                                      seed=self.seed, average=self.average,
                                      include_stale=self.include_stale, timeout_s=self.timeout_s,
                                      grace_us=self.grace_us, hyper=b.hyper, max_blocks=self.max_blocks,
                                      two_shot_min=self.two_shot_min, accumulate=self.accumulate,
                                      adaptive_grace=self.adaptive_grace, mc_base=arena.mc_base, **kw)
            self._refresh_hyper(b, force=True)
        if master_of:
            if len(self.optimizer.state) != 0:
                raise ValueError("wrap the optimizer before its first step: its state is keyed by the parameters, "
                                 "which are replaced by fp32 master copies here")
            for pg in self.optimizer.param_groups:
                pg["params"] = [master_of.get(id(p), p) for p in pg["params"]]
        torch.cuda.synchronize(self.device)
        g.barrier()

    def _lars_tables(self, b: _Bucket):
        """Chunk records (start, length, tensor) of one bucket for the fused LARS kernels: chunks never straddle
        a tensor; tensors the optimizer does not adapt (biases, batch-norm scale / shift) carry a negative index."""
        import ctypes as C
        lib = N.cuda()
        lib.esgd_lars_step.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_float,
                                       C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_float, C.c_float, C.c_float,
                                       C.c_float, C.c_void_p]
        chunk = int(lib.esgd_lars_chunk_elems())
        rec = []
        for t, (p, off) in enumerate(zip(b.params, b.offsets)):
            padded = (p.numel() + _PAD - 1) // _PAD * _PAD
            for s0 in range(0, padded, chunk):
                rec.append((off + s0, min(chunk, padded - s0), (-1 - t) if self.optimizer.skip(p) else t))
        arr = np.zeros(len(rec), dtype=np.dtype([("start", "<i8"), ("len", "<i4"), ("tensor", "<i4")]))
        for i, r in enumerate(rec):
            arr[i] = r
        b.lars_chunks = torch.from_numpy(arr.view(np.uint8).copy()).to(self.device)
        b.lars_num_chunks = len(rec)
        b.lars_sq = torch.zeros(2 * len(b.params), dtype=torch.float32, device=self.device)

    def _lars_step(self):
        s = torch.cuda.current_stream(self.device).cuda_stream
        for b in self.buckets:
            pg = self.optimizer.param_groups[b.group_index]
            N.check_cuda(N.cuda().esgd_lars_step(
                b.lars_chunks.data_ptr(), b.lars_num_chunks, len(b.params), b.lars_sq.data_ptr(), b.g32.data_ptr(), 0,
                float(self.grad_scale), b.w32.data_ptr(), b.mom.data_ptr(),
                b.w16.data_ptr() if b.w16 is not None else None, float(pg["lr"]), float(pg["momentum"]),
                float(pg["weight_decay"]), float(pg["eeta"]), float(pg["epsilon"]), s), "fused LARS step")

    def _refresh_hyper(self, b: _Bucket, force: bool = False):
        pg = self.optimizer.param_groups[b.group_index]
        vals = (float(pg.get("lr", 0.0)), float(pg.get("momentum", 0.0)), float(pg.get("weight_decay", 0.0)),
                bool(pg.get("nesterov", False)), float(getattr(self, "grad_scale", 1.0)))
        if force or vals != b.hyper_vals:
            if torch.cuda.is_current_stream_capturing():
                return  # a captured step reads the device copy; sync_hyper() refreshes it before a replay
            b.hyper_vals = vals
            # the values travel as launch arguments of a one-thread kernel on the current stream (the side
            # stream waits for it before every launch): a step always reads what was current when it was
            # enqueued, however far the host runs ahead of the GPU
            b.channel.set_hyper(*vals)

    def sync_hyper(self):
        """Push lr / momentum / weight decay to the device copies the fused kernels read.
        Needed before replaying a CUDA graph that contains ``step()``."""
        if self.on_gpu:
            for b in self.buckets:
                self._refresh_hyper(b)

    def refresh_master_from_params(self):
        """Re-derive the fp32 master weights (and the low-precision working copies) from the values the
        parameters hold now.  Call it after writing into the parameters from outside the optimizer — a
        warm start, a checkpoint without master weights — or the next update starts from the old masters."""
        if not self.on_gpu:
            return
        torch.cuda.current_stream(self.device).wait_stream(self.comm_stream)
        for b in self.buckets:
            if b.w32 is None:
                continue
            for p, off in zip(b.params, b.offsets):
                _view_like(b.w32, off, p).copy_(p.detach().float())

    def _install_hooks(self):
        for b in self.buckets:
            b.pending = len(b.params)
            for p in b.params:
                self._hooks.append(p.register_post_accumulate_grad_hook(self._make_hook(b)))

    def _make_hook(self, b: _Bucket):
        def hook(p):
            b.dirty = True
            b.pending -= 1
            if b.pending == 0 and self.overlap:
                self._launch(b)
        return hook

    def _launch(self, b: _Bucket):
        """Start the bucket's partial allreduce on the side stream, behind backward."""
        if b.launched:
            return
        for p, off in zip(b.params, b.offsets):  # a foreign .grad (zero_grad(set_to_none)) is copied back in
            if p.grad is not None and p.grad.data_ptr() != b.grad_flat.data_ptr() + off * b.grad_flat.element_size():
                _view_like(b.grad_flat, off, p).copy_(p.grad)
                p.grad = _view_like(b.grad_flat, off, p)
        self._refresh_hyper(b)
        self.comm_stream.wait_stream(torch.cuda.current_stream(self.device))
        with nvtx_range("partial_allreduce"):
            b.channel.step(self.comm_stream)
        b.launched = True

    # ------------------------------------------------------------------ API
    @property
    def param_groups(self):
        return self.optimizer.param_groups

    def zero_grad(self, set_to_none: bool = False):
        """Zero the flat gradient buckets (the per-parameter ``.grad`` stay views of them).  On the GPU
        the reduce kernel clears a bucket behind its copy into the publish slot, so after ``step()`` there
        is nothing left to do here; a fill is launched only for a bucket that backward has written since."""
        for b in self.buckets:
            if not (self.on_gpu and getattr(b, "self_clearing", False) and not b.dirty):
                b.grad_flat.zero_()
                if self.on_gpu:
                    b.dirty = False
            if any(p.grad is None for p in b.params):
                self._point_grads(b)

    def step(self, closure=None):
        loss = closure() if closure is not None else None
        self.steps += 1
        if self.on_gpu:
            for b in self.buckets:
                self._launch(b)
            torch.cuda.current_stream(self.device).wait_stream(self.comm_stream)
            for b in self.buckets:
                b.launched = False
                b.pending = len(b.params)
                b.dirty = not b.self_clearing
            if not self.fused:
                self._inner_step()
        else:
            applied = False
            for b in self.buckets:
                out, info = b.channel.step(b.grad_flat, b.out_np)
                b.grad_flat.copy_(torch.from_numpy(out))
                if self.grad_scale != 1.0:
                    b.grad_flat.mul_(self.grad_scale)
                applied = applied or info.role in (N.ROLE_PARTICIPANT, N.ROLE_DRAIN)
                b.last_role = info.role
            if applied:
                self.optimizer.step()
        return loss

    def _inner_step(self):
        """Step the wrapped optimizer with the averaged gradients the kernels wrote — unless no bucket had
        anything to apply (the rank missed the round and its mailbox was empty, or a bounded wait ran out):
        then momentum and weight decay must not move the weights either, as on the CPU path and in the
        fused kernel.  Reading the flags synchronises with the device; inside stream capture the step is
        recorded unconditionally."""
        if not torch.cuda.is_current_stream_capturing():
            if not any(b.channel.applied() for b in self.buckets):
                return
        if self.lars:
            return self._lars_step()
        if self.grad_scale != 1.0:
            for b in self.buckets:
                (b.g32 if b.masters is not None else b.grad_flat).mul_(self.grad_scale)
        self.optimizer.step()
        for b in self.buckets:
            if b.masters is not None:
                b.w16.copy_(b.w32)

    def flush(self):
        """Apply the results of rounds that completed after this rank's last step."""
        if self.on_gpu:
            self.comm_stream.wait_stream(torch.cuda.current_stream(self.device))
            for b in self.buckets:
                self._refresh_hyper(b)
                b.channel.flush(self.comm_stream)
            torch.cuda.current_stream(self.device).wait_stream(self.comm_stream)
            if not self.fused:
                self._inner_step()
        else:
            applied = False
            for b in self.buckets:
                out, info = b.channel.flush(b.out_np)
                b.grad_flat.copy_(torch.from_numpy(out))
                applied = applied or info.role == N.ROLE_DRAIN
            if applied:
                self.optimizer.step()

    def check(self):
        """Raise ``ChannelError`` if any bounded wait ran out (synchronises on GPU)."""
        for b in self.buckets:
            st = b.channel.stats()["status"]
            if st:
                raise N.ChannelError(st, "bucket %d rank %d" % (b.index, self.group.rank))

    def stats(self) -> dict:
        """Eager-specific counters: rounds taken part in / missed / opened, forced
        synchronous rounds, dropped gradients, mean contributors, wait time."""
        per = [b.channel.stats() for b in self.buckets]
        s0 = per[0]
        part = max(s0["participated"], 1)
        return {
            "steps": s0["local_step"], "participated": s0["participated"], "absent": s0["absent"],
            "activated": s0["activated"], "forced_sync": s0["sync_rounds"], "dropped_grads": s0["dropped_grads"],
            "folded_grads": s0.get("folded_grads", 0),
            "mean_contributors": s0["contrib_sum"] / part, "wait_ms": sum(p["wait_ns"] for p in per) / 1e6,
            "staleness": s0["latest_round"] - s0["last_round"] if s0["latest_round"] >= s0["last_round"] else 0,
            "status": max(p["status"] for p in per), "buckets": len(per),
        }

    def trace(self, bucket: int = 0) -> list:
        """Per-step trace of one bucket's channel (newest 64 steps): role, round, activator,
        fresh / contributor masks, time spent waiting."""
        return self.buckets[bucket].channel.trace()

    def dump_trace(self, path: str) -> None:
        import json
        with open(path, "w") as f:
            json.dump({"rank": self.group.rank, "mode": self.mode,
                       "buckets": [b.channel.trace() for b in self.buckets], "stats": self.stats()}, f)

    def master_params(self):
        """(parameter, fp32 master view) pairs of the fused path; (p, p) otherwise."""
        for b in self.buckets:
            for p, off in zip(b.params, b.offsets):
                yield p, (_view_like(b.w32, off, p) if b.w32 is not None else p.data)

    def momentum_buffers(self):
        for b in self.buckets:
            for p, off in zip(b.params, b.offsets):
                if b.mom is not None:
                    yield p, _view_like(b.mom, off, p)
                else:
                    key = b.masters[b.params.index(p)] if b.masters is not None else p
                    yield p, self.optimizer.state.get(key, {}).get("momentum_buffer")

    def state_dict(self) -> dict:
        sd = {"inner": self.optimizer.state_dict(), "steps": self.steps, "mode": self.mode,
              "limiter": self.limiter, "seed": self.seed}
        if self.fused or self.lars:
            sd["fused_master"] = [b.w32.detach().cpu() for b in self.buckets]
            sd["fused_momentum"] = [b.mom.detach().cpu() for b in self.buckets]
        return sd

    def load_state_dict(self, sd: dict):
        self.optimizer.load_state_dict(sd["inner"])
        self.steps = sd.get("steps", 0)
        if (self.fused or self.lars) and "fused_master" in sd:
            for b, w, m in zip(self.buckets, sd["fused_master"], sd["fused_momentum"]):
                b.w32.copy_(w)
                b.mom.copy_(m)
                if b.w16 is not None:
                    b.w16.copy_(b.w32)
        else:   # a checkpoint without master weights: the parameters as loaded are the truth
            self.refresh_master_from_params()

    def resync_from_rank0(self):
        """Overwrite this replica with rank 0's weights, momentum and (optionally
        diverged) buffers — the in-job form of the reference's checkpoint copy
        between launches (resnet/test_scripts_imagenet/synchm.sh:4-12)."""
        g = self.group
        if g.world == 1:
            return
        if self.on_gpu:
            torch.cuda.current_stream(self.device).wait_stream(self.comm_stream)
        for b in self.buckets:
            if self.fused or self.lars:
                g.bcast(b.w32)
                g.bcast(b.mom)
                if b.w16 is not None:
                    b.w16.copy_(b.w32)
            else:
                if b.masters is not None:
                    g.bcast(b.w32)
                    b.w16.copy_(b.w32)
                for p in (b.masters if b.masters is not None else b.params):
                    if b.masters is None:
                        g.bcast(p.data)
                    buf = self.optimizer.state.get(p, {}).get("momentum_buffer")
                    if buf is not None:
                        g.bcast(buf)

    def close(self):
        for h in self._hooks:
            h.remove()
        self._hooks = []
        if self.on_gpu:
            torch.cuda.synchronize(self.device)
            self.group.barrier()
            for a in getattr(self, "_arenas", []):
                a.free()
            self._arenas = []
        else:
            if self.group.world > 1:
                self.group.barrier()
            for s in getattr(self, "_segments", []):
                s.close()
            self._segments = []


class SoloAllreduceOptimizer(EagerOptimizer):
    """First arriver triggers the round; ``limiter`` eager rounds, then a synchronous one."""

    def __init__(self, optimizer, group=None, limiter: int = 32, **kw):
        super().__init__(optimizer, group, mode="solo", limiter=limiter, **kw)


class MajorityAllreduceOptimizer(EagerOptimizer):
    """A shared-seed pseudo-random initiator triggers each round."""

    def __init__(self, optimizer, group=None, seed: int = 6545343, limiter: int = -1, **kw):
        super().__init__(optimizer, group, mode="majority", limiter=limiter, seed=seed, **kw)


class SyncAllreduceOptimizer(EagerOptimizer):
    """Every round waits for every rank: synchronous data-parallel SGD."""

    def __init__(self, optimizer, group=None, **kw):
        kw.setdefault("average", "world")
        super().__init__(optimizer, group, mode="sync", limiter=-1, **kw)
