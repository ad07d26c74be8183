"""NVLink backend of the partial allreduce: peer-mapped arenas + sm_100a kernels.

Each rank allocates one arena per channel with ``cudaMalloc``
(``[control block | publish slot 0 | publish slot 1 | shard buffer | fp32 running sum]``), exports
it with a CUDA IPC handle and maps every peer's arena, so the kernels read and
write the other GPUs' memory directly over NVLink 5 / NVSwitch.  This replaces
the reference's buffers, pools and MPI transport (fflib2 src/ffbuffer.c,
src/ffstorage.c, src/components/mpi/*) and its progress thread: whoever takes
part in a round does the reduction itself with one-sided peer loads, so a rank
that has not arrived needs no agent running on its behalf.
"""
from __future__ import annotations

import ctypes as C
from typing import Callable, List, Optional

import torch

from . import _native as N

_MODES = {"solo": N.MODE_SOLO, "majority": N.MODE_MAJORITY, "sync": N.MODE_SYNC}
_AVG = {"contributors": N.AVG_CONTRIBUTORS, "world": N.AVG_WORLD, "sum": N.AVG_SUM}
HYPER_LEN = 8  # lr, momentum, weight_decay, nesterov, grad_scale, pad...
# Elements from which a round with several participants and at least three contributors is reduced in two
# shots (reduce-scatter by peer loads, then every participant pulls the other shares): below it the extra
# flag round trip costs more than the bytes it saves.
TWO_SHOT_MIN = 1 << 20
# Elements from which a round with every rank on time is reduced inside the NVSwitch (multimem), when the
# arenas have a multicast mapping.
MULTICAST_MIN = 1 << 12
# Bytes of a channel above which the multicast broadcast is not used: stores through the switch into eight arenas
# ran at 340 GB/s, so from here peer loads are the faster gather (8 GPUs, 256 MiB: 776 against 899 us).
MULTICAST_MAX_BYTES = 64 << 20
GUARD_BYTES = 256
GUARD_VALUE = 0xA5
_FLOAT_DTYPES = (torch.float32, torch.bfloat16)


def _check_dtype(t: Optional[torch.Tensor], what: str, allowed=_FLOAT_DTYPES) -> None:
    if t is not None and t.dtype not in allowed:
        raise ValueError("%s must be %s, not %s: the kernels of the partial allreduce read and write float32 and "
                         "bfloat16 only" % (what, " or ".join(str(a) for a in allowed), t.dtype))


def _align(x: int, a: int = 256) -> int:
    return (x + a - 1) // a * a


class ArenaLayout:
    def __init__(self, count: int, slot_dtype: torch.dtype):
        if count % 8:
            raise ValueError("channel element count must be a multiple of 8")
        esz = 2 if slot_dtype == torch.bfloat16 else 4
        # [control | guard | slot 0 | guard | slot 1 | guard | shard buffer | guard | running sum | guard]: the
        # guards hold a fixed pattern that no kernel ever writes; check_canaries() finds an overrun of a
        # neighbouring region (the debugging aid that stands in for a memory checker on shared GPUs)
        self.guards = []
        off = _align(int(N.cuda().esgd_dev_ctl_bytes()))

        def guard():
            nonlocal off
            self.guards.append(off)
            off += GUARD_BYTES

        self.ctl = 0
        guard()
        self.slot0 = off
        off += _align(count * esz)
        guard()
        self.slot1 = off
        off += _align(count * esz)
        guard()
        self.red = off
        off += _align(count * esz)
        guard()
        self.rsum = off
        off += _align(count * 4)
        guard()
        self.total = off


class Arena:
    """One cudaMalloc'd, zeroed, IPC-exportable allocation on the current device."""

    def __init__(self, nbytes: int, export: bool = True):
        self.mc_base = 0
        self.ptr = C.c_void_p()
        self.handle = (C.c_ubyte * 64)()
        N.check_cuda(N.cuda().esgd_arena_alloc(nbytes, C.byref(self.ptr), self.handle if export else None),
                     "arena allocation")
        self.nbytes = nbytes
        self.base = int(self.ptr.value)

    def free(self):
        if self.ptr:
            N.cuda().esgd_arena_free(self.ptr)
            self.ptr = C.c_void_p()


class _DevicePointer:
    """Lets ``torch.as_tensor`` wrap device memory this package allocated itself (CUDA array interface)."""

    def __init__(self, ptr: int, count: int, dtype: torch.dtype, keep=None):
        typestr = {torch.float32: "<f4", torch.bfloat16: "<u2", torch.uint8: "|u1"}[dtype]
        self.__cuda_array_interface__ = {"shape": (count,), "typestr": typestr, "data": (ptr, False), "version": 3}
        self.keep = keep


def device_view(ptr: int, count: int, dtype: torch.dtype, device: torch.device, keep=None) -> torch.Tensor:
    t = torch.as_tensor(_DevicePointer(ptr, count, dtype, keep), device=device)
    return t.view(torch.bfloat16) if dtype == torch.bfloat16 else t


class SymmetricArena:
    """An arena in symmetric memory with an NVLink multicast mapping (NVSwitch): ``bases`` are the ranks'
    peer-mapped addresses of it and ``mc_base`` is ONE address whose loads reduce over, and whose stores
    land in, every rank's copy (``multimem`` instructions).  Allocation, handle exchange and the multicast
    binding are PyTorch's symmetric-memory plumbing; every kernel that touches the memory is this package's."""

    def __init__(self, nbytes: int, device: torch.device, group_name: str):
        import torch.distributed._symmetric_memory as symm
        self.tensor = symm.empty(nbytes, dtype=torch.uint8, device=device)
        self.tensor.zero_()
        torch.cuda.synchronize(device)
        self.handle = symm.rendezvous(self.tensor, group_name)
        self.bases = [int(p) for p in self.handle.buffer_ptrs]
        self.mc_base = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        self.nbytes = nbytes
        self.base = int(self.tensor.data_ptr())

    def free(self):
        self.handle = None
        self.tensor = None


def multicast_wanted() -> bool:
    """NVSwitch multicast is used unless it is switched off: ``ESGD_MULTICAST=0``, or ``NCCL_NVLS_ENABLE=0``
    (one switch for every library of a job — tests in which a rank leaves a running job set it, because memory
    bound to a multicast object must not lose its owner)."""
    import os
    return os.environ.get("ESGD_MULTICAST", "1") != "0" and os.environ.get("NCCL_NVLS_ENABLE", "1") != "0"


def open_peer(handle_bytes: bytes) -> int:
    buf = (C.c_ubyte * 64).from_buffer_copy(handle_bytes)
    ptr = C.c_void_p()
    N.check_cuda(N.cuda().esgd_arena_open(buf, C.byref(ptr)), "opening a peer arena (CUDA IPC)")
    return int(ptr.value)


class NvlinkChannel:
    """One persistent partial-allreduce channel of ``count`` elements on this GPU.

    ``grad_in`` is the flat gradient the backward pass writes; ``None`` selects zero-copy publishing: the
    caller writes each step's gradient straight into ``publish_view()`` (this rank's publish slot of the
    coming epoch, in peer-mapped memory) and no staging copy runs.  With ``w32``/
    ``mom`` (and optionally ``w16``) the reduction is fused with the momentum-SGD
    update; otherwise the averaged gradient is written to ``out``.

    Channels of at least ``two_shot_min`` elements reduce in two shots when a round has
    several participants and at least three contributors (each participant sums its share,
    then pulls the others' shares); ``two_shot_min=None`` keeps the one-shot form.
    With ``mc_base`` (the multicast address of arenas from ``create_arenas``) rounds in which every rank is
    on time are reduced inside the NVSwitch from ``mc_min`` elements up.
    ``accumulate`` folds a gradient that no round picked up into the rank's next publish of
    the same slot instead of dropping it; ``clear_grad`` zeroes ``grad_in`` behind the copy
    into the publish slot, so the caller needs no separate fill before the next backward.
    """

    def __init__(self, count: int, rank: int, world: int, bases: List[int], device: torch.device,
                 grad_in: torch.Tensor, slot_dtype: torch.dtype = torch.bfloat16, mode: str = "solo",
                 limiter: int = 32, seed: int = 6545343, average: str = "contributors",
                 include_stale: bool = True, timeout_s: float = 20.0, grace_us: float = 50.0, home: int = 0,
                 w32: Optional[torch.Tensor] = None, mom: Optional[torch.Tensor] = None,
                 w16: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                 hyper: Optional[torch.Tensor] = None, max_blocks: int = 592,
                 two_shot_min: Optional[int] = TWO_SHOT_MIN, accumulate: bool = False,
                 adaptive_grace: bool = True, clear_grad: bool = False, mc_base: int = 0,
                 mc_min: int = MULTICAST_MIN):
        if slot_dtype not in _FLOAT_DTYPES:
            raise ValueError("slot_dtype must be torch.float32 or torch.bfloat16, not %s" % slot_dtype)
        _check_dtype(grad_in, "grad_in")
        if grad_in is None and accumulate:
            raise ValueError("zero-copy publishing overwrites the slot: it cannot fold an older gradient in")
        _check_dtype(w32, "w32", (torch.float32,))
        _check_dtype(mom, "mom", (torch.float32,))
        _check_dtype(w16, "w16", (torch.bfloat16,))
        _check_dtype(out, "out")
        for name, t in (("w32", w32), ("mom", mom), ("w16", w16), ("out", out)):
            if t is not None and (t.numel() != count or not t.is_contiguous()):
                raise ValueError("%s must be a contiguous tensor of %d elements" % (name, count))
        self.lib = N.cuda()
        self.count, self.rank, self.world, self.device = count, rank, world, device
        self.max_blocks = max_blocks
        self.layout = ArenaLayout(count, slot_dtype)
        self.bases = list(bases)
        self.grad_in, self.w32, self.mom, self.w16, self.out = grad_in, w32, mom, w16, out
        if hyper is None:
            hyper = torch.zeros(HYPER_LEN, dtype=torch.float32, device=device)
            hyper[4] = 1.0
        self.hyper = hyper
        assert grad_in is None or (grad_in.numel() == count and grad_in.is_contiguous())
        self.slot_dtype = slot_dtype
        self._steps = 0
        self._dch = torch.zeros(int(self.lib.esgd_dev_channel_bytes()), dtype=torch.uint8, device=device)
        d = N.ChannelDesc()
        L = self.layout
        for j in range(world):
            d.ctl[j] = bases[j] + L.ctl
            d.slot0[j] = bases[j] + L.slot0
            d.slot1[j] = bases[j] + L.slot1
            d.red[j] = bases[j] + L.red if two_shot_min is not None else None
            d.rsum[j] = bases[j] + L.rsum
        if mc_base and count * (2 if slot_dtype == torch.bfloat16 else 4) > MULTICAST_MAX_BYTES:
            mc_base = 0
        if mc_base and two_shot_min is not None and world > 1:
            d.mc_slot0, d.mc_slot1, d.mc_red = mc_base + L.slot0, mc_base + L.slot1, mc_base + L.red
            d.mc_min = max(int(mc_min), int(two_shot_min))      # never where one shot is the faster form
        self.multicast = bool(mc_base and two_shot_min is not None and world > 1)
        d.two_shot_min = int(two_shot_min) if two_shot_min is not None else 0
        d.accumulate, d.adaptive_grace, d.clear_grad = int(accumulate), int(adaptive_grace), int(clear_grad)
        self.two_shot = int(two_shot_min is not None and world >= 2 and count >= two_shot_min)
        d.rank, d.world, d.base_mode = rank, world, _MODES[mode]
        d.include_stale, d.average, d.home = int(include_stale), _AVG[average], home
        d.slot_bf16 = int(slot_dtype == torch.bfloat16)
        d.grad_in_bf16 = int(grad_in is not None and grad_in.dtype == torch.bfloat16)
        d.limiter, d.seed = limiter, seed
        d.timeout_ns, d.grace_ns, d.count = int(timeout_s * 1e9), int(grace_us * 1e3), count
        d.grad_in = grad_in.data_ptr() if grad_in is not None else None
        d.w32 = w32.data_ptr() if w32 is not None else None
        d.mom = mom.data_ptr() if mom is not None else None
        d.w16 = w16.data_ptr() if w16 is not None else None
        d.out = out.data_ptr() if out is not None else None
        d.out_bf16 = int(out is not None and out.dtype == torch.bfloat16)
        d.hyper = self.hyper.data_ptr()
        self._desc = d
        stream = torch.cuda.current_stream(device)
        N.check_cuda(self.lib.esgd_channel_configure(self._dch.data_ptr(), C.byref(d), stream.cuda_stream),
                     "channel configuration")
        self._ctl_host = (C.c_ubyte * int(self.lib.esgd_dev_ctl_bytes()))()
        for g in self.layout.guards:     # this rank's own arena; peers paint theirs
            device_view(self.bases[self.rank] + g, GUARD_BYTES, torch.uint8, device).fill_(GUARD_VALUE)

    @property
    def dev_ptr(self) -> int:
        return self._dch.data_ptr()

    def step(self, stream: Optional[torch.cuda.Stream] = None) -> None:
        """Enqueue one step on ``stream``: pack + control, then reduce + update."""
        s = stream if stream is not None else torch.cuda.current_stream(self.device)
        N.check_cuda(self.lib.esgd_channel_step(self._dch.data_ptr(), self.count, self.max_blocks, s.cuda_stream),
                     "partial allreduce launch")
        self._steps += 1

    def publish_view(self) -> torch.Tensor:
        """This rank's publish slot of the coming step as a tensor (zero-copy publishing: fill it, then ``step()``).
        Slots alternate from step to step; a slot is free again once the step after next is being prepared, which
        ``step()`` checks on the device — do not write into a view obtained before the previous ``step()``."""
        parity = (self._steps + 1) % 2
        off = self.layout.slot0 if parity == 0 else self.layout.slot1
        return device_view(self.bases[self.rank] + off, self.count, self.slot_dtype, self.device)

    def set_hyper(self, lr: float, momentum: float, weight_decay: float, nesterov: bool, grad_scale: float,
                  stream: Optional[torch.cuda.Stream] = None) -> None:
        """Enqueue new hyper-parameters on ``stream``; steps enqueued later on streams that wait for it read them."""
        s = stream if stream is not None else torch.cuda.current_stream(self.device)
        N.check_cuda(self.lib.esgd_set_hyper(self.hyper.data_ptr(), lr, momentum, weight_decay, int(nesterov),
                                             grad_scale, s.cuda_stream), "hyper-parameter update")

    def check_canaries(self) -> None:
        """Raise if any guard region between the sections of this rank's arena no longer holds its pattern: some
        kernel, local or on a peer, wrote past the end (or before the start) of a slot, the shard buffer or the
        running sum.  Synchronises with the device."""
        torch.cuda.synchronize(self.device)
        for k, g in enumerate(self.layout.guards):
            v = device_view(self.bases[self.rank] + g, GUARD_BYTES, torch.uint8, self.device)
            if not bool((v == GUARD_VALUE).all()):
                bad = int((v != GUARD_VALUE).nonzero()[0])
                raise RuntimeError("arena guard %d of rank %d was overwritten at byte %d: a kernel wrote outside its "
                                   "region" % (k, self.rank, bad))

    def applied(self) -> bool:
        """Whether the newest step applied anything (it took part in a round or collected missed ones).
        Synchronises with the current stream."""
        v = C.c_int(0)
        s = torch.cuda.current_stream(self.device)
        N.check_cuda(self.lib.esgd_channel_applied(self._dch.data_ptr(), C.byref(v), s.cuda_stream),
                     "reading the step's outcome")
        return bool(v.value)

    def phase_times_us(self) -> dict:
        """Where the newest step spent its time on the device (microseconds): packing, the control step
        (publish, election, waits, descriptor), the gap to the data kernel, the data phase.  Synchronises."""
        t = (C.c_uint64 * 8)()
        s = torch.cuda.current_stream(self.device)
        N.check_cuda(self.lib.esgd_channel_times(self._dch.data_ptr(), t, s.cuda_stream), "reading phase clocks")
        us = lambda a, b: (int(t[b]) - int(t[a])) / 1e3
        return {"pack": us(0, 1), "control": us(1, 2), "launch_gap": us(2, 3), "data": us(3, 5),
                "own_share": us(3, 4) if t[4] >= t[3] else None}

    def flush(self, stream: Optional[torch.cuda.Stream] = None) -> None:
        s = stream if stream is not None else torch.cuda.current_stream(self.device)
        N.check_cuda(self.lib.esgd_channel_flush(self._dch.data_ptr(), self.count, self.max_blocks, s.cuda_stream),
                     "partial allreduce flush launch")

    def stats(self) -> dict:
        """Synchronising read of this rank's counters and sticky status word."""
        s = torch.cuda.current_stream(self.device)
        N.check_cuda(self.lib.esgd_memcpy_d2h(self._ctl_host, C.c_void_p(self.bases[self.rank] + self.layout.ctl),
                                              len(self._ctl_host), s.cuda_stream), "reading channel counters")
        raw = (C.c_uint64 * 24)()
        N.host().esgd_ctl_stats(self._ctl_host, raw)
        return N.parse_stats(raw)

    def trace(self) -> list:
        """The newest (up to 64) steps of this rank: role, round, activator, masks, wait time."""
        self.stats()   # refreshes the host copy of the control block
        return N.parse_trace(self._ctl_host)

    def check(self, where: str = "") -> None:
        st = self.stats()["status"]
        if st:
            raise N.ChannelError(st, where or "gpu rank %d" % self.rank)


def create_arenas(count: int, slot_dtype: torch.dtype, rank: int, world: int,
                  exchange: Optional[Callable] = None, multicast: Optional[bool] = None):
    """Allocate this rank's arena and map the peers'.  Returns (own arena, bases); ``arena.mc_base`` is the
    arena's NVLink multicast address, or 0.  With ``multicast`` (default: ``multicast_wanted()``) and an
    initialised NCCL process group the arena comes from symmetric memory; if any rank cannot get that, all
    ranks fall back to ``cudaMalloc`` + CUDA IPC."""
    layout = ArenaLayout(count, slot_dtype)
    if world == 1:
        arena = Arena(layout.total, export=False)
        return arena, [arena.base]
    import torch.distributed as dist
    if multicast is None:
        multicast = multicast_wanted()
    want = bool(multicast and dist.is_available() and dist.is_initialized() and dist.get_backend() == "nccl" and
                dist.get_world_size() == world)
    if all(exchange(want)):
        arena, err = None, ""
        try:
            arena = SymmetricArena(layout.total, torch.device("cuda", torch.cuda.current_device()),
                                   dist.group.WORLD.group_name)
        except Exception as e:  # noqa
            err = repr(e)[:200]
        oks = exchange(arena is not None and arena.mc_base != 0)
        if all(oks):
            exchange("mapped")
            return arena, arena.bases
        if arena is not None:
            arena.free()
        if rank == 0:
            import warnings
            warnings.warn("no NVLink multicast arena (%s): using CUDA IPC arenas" % (err or "a rank has none"))
    arena = Arena(layout.total, export=True)
    handles = exchange(bytes(arena.handle))
    bases = [arena.base if r == rank else open_peer(h) for r, h in enumerate(handles)]
    exchange("mapped")
    return arena, bases


class EmulatedWorld:
    """``world`` ranks of one channel on ONE GPU, stepped by a single cooperative
    launch (one block per rank).  Exercises the device protocol, the peer-pointer
    data path and the mailbox on a single-GPU box."""

    def __init__(self, world: int, count: int, device: torch.device, slot_dtype=torch.bfloat16,
                 grad_dtype=torch.float32, fused: bool = False, **kw):
        self.world, self.count, self.device = world, count, device
        layout = ArenaLayout(count, slot_dtype)
        self.arenas = [Arena(layout.total, export=False) for _ in range(world)]
        bases = [a.base for a in self.arenas]
        self.grads = [torch.zeros(count, dtype=grad_dtype, device=device) for _ in range(world)]
        self.outs = [torch.zeros(count, dtype=torch.float32, device=device) for _ in range(world)]
        self.w32 = [torch.zeros(count, dtype=torch.float32, device=device) for _ in range(world)] if fused else None
        self.mom = [torch.zeros(count, dtype=torch.float32, device=device) for _ in range(world)] if fused else None
        self.w16 = [torch.zeros(count, dtype=torch.bfloat16, device=device) for _ in range(world)] if fused else None
        self.hyper = torch.zeros(HYPER_LEN, dtype=torch.float32, device=device)
        self.hyper[4] = 1.0
        self.channels = []
        for r in range(world):
            self.channels.append(NvlinkChannel(
                count, r, world, bases, device, self.grads[r], slot_dtype=slot_dtype,
                w32=self.w32[r] if fused else None, mom=self.mom[r] if fused else None,
                w16=self.w16[r] if fused else None, out=None if fused else self.outs[r], hyper=self.hyper, **kw))
        self._chans = torch.tensor([c.dev_ptr for c in self.channels], dtype=torch.int64, device=device)
        self._delays = torch.zeros(world, dtype=torch.int64, device=device)

    def step(self, delays_us=None, flush: bool = False) -> None:
        if delays_us is not None:
            self._delays.copy_(torch.tensor([int(d * 1000) for d in delays_us], dtype=torch.int64))
        else:
            self._delays.zero_()
        s = torch.cuda.current_stream(self.device)
        N.check_cuda(N.cuda().esgd_emulated_step(self._chans.data_ptr(), self._delays.data_ptr(), self.world,
                                                 int(flush), s.cuda_stream), "emulated multi-rank step")

    def close(self):
        torch.cuda.synchronize(self.device)
        for a in self.arenas:
            a.free()
