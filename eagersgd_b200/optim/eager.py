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
        self.w32 = self.mom = self.w16 = None
        self.hyper = None
        self.hyper_host = None
        self.hyper_vals = None

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
                 grace_us: float = 50.0, max_blocks: int = 592, two_shot_min: Optional[int] = 1 << 26,
                 two_shot_parts: int = 5):
        self.optimizer = optimizer
        self.two_shot_min = two_shot_min   # bucket elements from which a round is reduced in two shots (None: never)
        self.two_shot_parts = two_shot_parts   # ... when at least this many ranks take part in it
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
        can_fuse = (self.on_gpu and type(optimizer) is torch.optim.SGD and
                    all(g.get("dampening", 0) == 0 and not g.get("maximize", False) for g in optimizer.param_groups))
        self.fused = can_fuse if fused is None else (fused and can_fuse)
        if slot_dtype is None:
            slot_dtype = torch.bfloat16 if params[0].dtype == torch.bfloat16 else torch.float32
        self.slot_dtype = slot_dtype
        self._build_buckets(bucket_mb)
        self._hooks = []
        if self.on_gpu:
            self._setup_gpu()
            if overlap:
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
                                   grace_us=self.grace_us)
            b.out_np = np.empty(b.count, dtype=npdt)

    # ------------------------------------------------------------------ GPU
    def _setup_gpu(self):
        from ..parallel.nvlink_channel import HYPER_LEN, NvlinkChannel, create_arenas
        g = self.group
        self.comm_stream = torch.cuda.Stream(device=self.device, priority=-1)
        self._arenas = []
        for b in self.buckets:
            dt = b.params[0].dtype
            b.grad_flat = torch.zeros(b.count, dtype=dt, device=self.device)
            b.hyper = torch.zeros(HYPER_LEN, dtype=torch.float32, device=self.device)
            b.hyper_host = torch.zeros(HYPER_LEN, dtype=torch.float32).pin_memory()
            kw = {}
            if self.fused:
                b.w32 = torch.zeros(b.count, dtype=torch.float32, device=self.device)
                b.mom = torch.zeros(b.count, dtype=torch.float32, device=self.device)
                if dt != torch.float32:
                    b.w16 = torch.zeros(b.count, dtype=dt, device=self.device)
                for p, off in zip(b.params, b.offsets):
                    _view_like(b.w32, off, p).copy_(p.detach().float())
                    store = b.w16 if b.w16 is not None else b.w32
                    v = _view_like(store, off, p)
                    if b.w16 is not None:
                        v.copy_(p.detach())
                    p.data = v  # the model now computes on the bucket's storage
                kw = dict(w32=b.w32, mom=b.mom, w16=b.w16)
            else:
                kw = dict(out=b.grad_flat)
            self._point_grads(b)
            arena, bases = create_arenas(b.count, self.slot_dtype, g.rank, g.world, g.exchange)
            self._arenas.append(arena)
            b.channel = NvlinkChannel(b.count, g.rank, g.world, bases, self.device, b.grad_flat,
                                      slot_dtype=self.slot_dtype, mode=self.mode, limiter=self.limiter,
                                      seed=self.seed, average=self.average,
                                      include_stale=self.include_stale, timeout_s=self.timeout_s,
                                      grace_us=self.grace_us, hyper=b.hyper, max_blocks=self.max_blocks,
                                      two_shot_min=self.two_shot_min, two_shot_parts=self.two_shot_parts, **kw)
            self._refresh_hyper(b, force=True)
        torch.cuda.synchronize(self.device)
        g.barrier()

    def _refresh_hyper(self, b: _Bucket, force: bool = False):
        pg = self.optimizer.param_groups[b.group_index]
        vals = (float(pg.get("lr", 0.0)), float(pg.get("momentum", 0.0)), float(pg.get("weight_decay", 0.0)),
                1.0 if pg.get("nesterov", False) else 0.0, float(getattr(self, "grad_scale", 1.0)))
        if force or vals != b.hyper_vals:
            if torch.cuda.is_current_stream_capturing():
                return  # a captured step reads the device copy; sync_hyper() refreshes it before a replay
            b.hyper_vals = vals
            for i, v in enumerate(vals):
                b.hyper_host[i] = v
            # on the current stream: the side stream waits for it before every launch
            b.hyper.copy_(b.hyper_host, non_blocking=True)

    def sync_hyper(self):
        """Push lr / momentum / weight decay to the device copies the fused kernels read.
        Needed before replaying a CUDA graph that contains ``step()``."""
        if self.on_gpu:
            for b in self.buckets:
                self._refresh_hyper(b)

    def _install_hooks(self):
        for b in self.buckets:
            b.pending = len(b.params)
            for p in b.params:
                self._hooks.append(p.register_post_accumulate_grad_hook(self._make_hook(b)))

    def _make_hook(self, b: _Bucket):
        def hook(p):
            b.pending -= 1
            if b.pending == 0:
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
        b.channel.step(self.comm_stream)
        b.launched = True

    # ------------------------------------------------------------------ API
    @property
    def param_groups(self):
        return self.optimizer.param_groups

    def zero_grad(self, set_to_none: bool = False):
        """Zero the flat gradient buckets (the per-parameter ``.grad`` stay views of them)."""
        for b in self.buckets:
            b.grad_flat.zero_()
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
            if not self.fused:
                if self.grad_scale != 1.0:
                    for b in self.buckets:
                        b.grad_flat.mul_(self.grad_scale)
                self.optimizer.step()
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

    def flush(self):
        """Apply the results of rounds that completed after this rank's last step."""
        if self.on_gpu:
            self.comm_stream.wait_stream(torch.cuda.current_stream(self.device))
            for b in self.buckets:
                self._refresh_hyper(b)
                b.channel.flush(self.comm_stream)
            torch.cuda.current_stream(self.device).wait_stream(self.comm_stream)
            if not self.fused:
                self.optimizer.step()
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
                    st = self.optimizer.state.get(p, {})
                    yield p, st.get("momentum_buffer")

    def state_dict(self) -> dict:
        sd = {"inner": self.optimizer.state_dict(), "steps": self.steps, "mode": self.mode,
              "limiter": self.limiter, "seed": self.seed}
        if self.fused:
            sd["fused_master"] = [b.w32.detach().cpu() for b in self.buckets]
            sd["fused_momentum"] = [b.mom.detach().cpu() for b in self.buckets]
        return sd

    def load_state_dict(self, sd: dict):
        self.optimizer.load_state_dict(sd["inner"])
        self.steps = sd.get("steps", 0)
        if self.fused and "fused_master" in sd:
            for b, w, m in zip(self.buckets, sd["fused_master"], sd["fused_momentum"]):
                b.w32.copy_(w)
                b.mom.copy_(m)
                if b.w16 is not None:
                    b.w16.copy_(b.w32)

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
            if self.fused:
                g.bcast(b.w32)
                g.bcast(b.mom)
                if b.w16 is not None:
                    b.w16.copy_(b.w32)
            else:
                for p in b.params:
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
