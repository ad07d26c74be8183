"""Broadcast, gather, all-gather, send / receive, barrier, all-reduce and the ring-neighbour sum as kernels of
this package over peer-mapped GPU memory (``csrc/cuda/peer_collectives.cu``).

GPU-native counterpart of the MPI operators the reference ships for its Caffe2 backend
(deep500/frameworks/caffe2/custom_operators/mpi/*.cpp) and of ``CommunicationNetwork``
(deep500/lv3/communication.py:14-119).  A source copies its tensor into its stage buffer and raises a counter
in each destination; a destination pulls the bytes over NVLink and acknowledges.  Calls must be made in the
same order by the ranks they involve (MPI semantics on one communicator); a tensor larger than the stage is
moved in pieces.  Every device wait is bounded: ``check()`` raises ``CollectiveError`` when one ran out.

``PeerCollectives`` is for one process per GPU; ``EmulatedCollectives`` runs all ranks on one GPU with one
cooperative launch per operation (kernels that wait on one another are never separate launches on one GPU).
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import torch

from . import _native as N
from .nvlink_channel import Arena, _align, open_peer

RED_NONE, RED_SUM_F32, RED_SUM_BF16 = 0, 1, 2
COLLECTIVE, POINT_TO_POINT = 0, 1      # classes of traffic: each has its own message counters per pair of ranks
_STATUS = {1: "a destination never acknowledged the previous message", 2: "a source never published"}


class CollectiveError(RuntimeError):
    pass


def _lib():
    lib = N.cuda()
    if not getattr(lib, "_coll_ready", False):
        lib.esgd_coll_ctl_bytes.restype = C.c_uint64
        lib.esgd_coll_rank_bytes.restype = C.c_uint64
        lib.esgd_coll_op_bytes.restype = C.c_uint64
        lib.esgd_coll_init.argtypes = [C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_uint64), C.c_uint64, C.c_double,
                                       C.c_void_p]
        lib.esgd_coll_exchange.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_int64, C.c_void_p, C.c_void_p,
                                           C.c_int64, C.c_int, C.c_int, C.c_int, C.c_void_p]
        lib.esgd_coll_exchange_emulated.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
        lib.esgd_coll_pack_op.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_int64, C.c_void_p, C.c_void_p,
                                          C.c_int64, C.c_int, C.c_int, C.c_int]
        lib.esgd_coll_probe.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p]
        lib.esgd_coll_state.argtypes = [C.c_void_p, C.POINTER(C.c_uint32), C.POINTER(C.c_int32), C.c_void_p]
        lib._coll_ready = True
    return lib


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _reduce_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return RED_SUM_F32
    if t.dtype == torch.bfloat16:
        return RED_SUM_BF16
    raise ValueError("the peer all-reduce sums float32 and bfloat16 tensors, not %s" % t.dtype)


def _flat(t: torch.Tensor) -> torch.Tensor:
    if not t.is_contiguous():
        raise ValueError("peer collectives take contiguous tensors")
    return t.view(-1).view(torch.uint8)


class _Plan:
    """The masks of each collective, for one rank of ``world``: what it publishes to and reads from."""

    def __init__(self, rank: int, world: int):
        self.rank, self.world = rank, world
        self.all = (1 << world) - 1
        self.others = self.all & ~(1 << rank)

    def bcast(self, root: int):
        return (self.others, 0, -1) if self.rank == root else (0, 1 << root, -1)

    def gather(self, root: int):
        dst = 0 if self.rank == root else 1 << root
        src = self.others if self.rank == root else 0
        return dst, src, (self.rank if self.rank == root else -1)

    def allgather(self):
        return self.others, self.others, self.rank

    def neighbours(self):
        left, right = (self.rank - 1) % self.world, (self.rank + 1) % self.world
        m = ((1 << left) | (1 << right)) & ~(1 << self.rank)
        return m, m, self.rank


class PeerCollectives:
    """Collectives of one rank (one process per GPU).  ``exchange`` all-gathers a small Python object between the
    ranks (used once, for the CUDA IPC handles)."""

    def __init__(self, rank: int, world: int, exchange, stage_mb: float = 64.0, timeout_s: float = 30.0,
                 device: Optional[torch.device] = None):
        lib = _lib()
        self.rank, self.world = rank, world
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.plan = _Plan(rank, world)
        self.stage_bytes = _align(int(stage_mb * (1 << 20)), 256)
        self.stage_off = _align(int(lib.esgd_coll_ctl_bytes()), 256)
        self.arena = Arena(self.stage_off + self.stage_bytes, export=world > 1)
        if world > 1:
            handles = exchange(bytes(self.arena.handle))
            self.bases = [self.arena.base if r == rank else open_peer(h) for r, h in enumerate(handles)]
            exchange("mapped")
        else:
            self.bases = [self.arena.base]
        self.desc = torch.zeros(int(lib.esgd_coll_rank_bytes()), dtype=torch.uint8, device=self.device)
        bases = (C.c_uint64 * world)(*self.bases)
        N.check_cuda(lib.esgd_coll_init(self.desc.data_ptr(), rank, world, bases, self.stage_off, timeout_s, _stream()),
                     "collective descriptor")

    # ---- one exchange, in pieces no larger than the stage ---------------------------------------------------
    def _exchange(self, dst: int, src: int, t_in: Optional[torch.Tensor], t_out: Optional[torch.Tensor], nbytes: int,
                  out_stride: int = 0, reduce: int = RED_NONE, self_slot: int = -1, cls: int = COLLECTIVE) -> None:
        lib = _lib()
        step = self.stage_bytes
        off = 0
        while True:
            n = min(step, nbytes - off)
            pin = t_in.data_ptr() + off if t_in is not None else 0
            pout = t_out.data_ptr() + off if t_out is not None else 0
            N.check_cuda(lib.esgd_coll_exchange(self.desc.data_ptr(), dst, src, n, pin, pout, out_stride, reduce,
                                                self_slot, cls, _stream()), "peer collective")
            off += n
            if off >= nbytes:
                break

    # ---- the collectives -----------------------------------------------------------------------------------------
    def barrier(self) -> None:
        self._exchange(self.plan.others, self.plan.others, None, None, 0)

    def bcast(self, t: torch.Tensor, root: int = 0) -> torch.Tensor:
        b = _flat(t)
        dst, src, _ = self.plan.bcast(root)
        self._exchange(dst, src, b, b, b.numel())
        return t

    def gather(self, t: torch.Tensor, root: int = 0) -> Optional[torch.Tensor]:
        """Root gets a tensor of shape (world, *t.shape); the others None."""
        b = _flat(t)
        dst, src, slot = self.plan.gather(root)
        out = torch.empty((self.world,) + tuple(t.shape), dtype=t.dtype, device=t.device) if self.rank == root else None
        self._gathering(dst, src, slot, b, out)
        return out

    def allgather(self, t: torch.Tensor) -> torch.Tensor:
        b = _flat(t)
        dst, src, slot = self.plan.allgather()
        out = torch.empty((self.world,) + tuple(t.shape), dtype=t.dtype, device=t.device)
        self._gathering(dst, src, slot, b, out)
        return out

    def _gathering(self, dst, src, slot, b, out):
        n = b.numel()
        if n <= self.stage_bytes:
            self._exchange(dst, src, b, _flat(out) if out is not None else None, n, out_stride=n, self_slot=slot)
            return
        # pieces: piece p of every source lands at out[j, p * stage : ...]; the stride between sources stays n
        lib = _lib()
        ob = _flat(out) if out is not None else None
        for off in range(0, n, self.stage_bytes):
            m = min(self.stage_bytes, n - off)
            N.check_cuda(lib.esgd_coll_exchange(self.desc.data_ptr(), dst, src, m, b.data_ptr() + off,
                                                ob.data_ptr() + off if ob is not None else 0, n, RED_NONE, slot,
                                                COLLECTIVE, _stream()), "peer gather")

    def send(self, t: torch.Tensor, dst: int) -> None:
        b = _flat(t)
        self._exchange(1 << dst, 0, b, None, b.numel(), cls=POINT_TO_POINT)

    def recv(self, t: torch.Tensor, src: int) -> int:
        b = _flat(t)
        self._exchange(0, 1 << src, None, b, b.numel(), cls=POINT_TO_POINT)
        return src

    def recv_any(self, t: torch.Tensor) -> int:
        """Receive from whichever rank has sent (point-to-point) first; returns its rank.  Synchronises the stream.
        Only ``send`` traffic is looked at, so a peer that has gone on to its next collective is never mistaken
        for a sender."""
        lib = _lib()
        N.check_cuda(lib.esgd_coll_probe(self.desc.data_ptr(), self.plan.others, _stream()), "probe")
        status, src = self._state()
        if src < 0:
            raise CollectiveError("no rank sent anything within the time limit")
        return self.recv(t, src)

    def allreduce(self, t: torch.Tensor, average: bool = False) -> torch.Tensor:
        """In-place sum over the ranks, added in rank order on every rank (identical bits everywhere)."""
        b = _flat(t)
        if b.numel() % 16 or b.data_ptr() % 16:
            self._reject(b)
        self._exchange(self.plan.others, self.plan.others, b, b, b.numel(), reduce=_reduce_code(t), self_slot=self.rank)
        if average:
            t.div_(self.world)
        return t

    @staticmethod
    def _reject(b):
        raise ValueError("the peer all-reduce needs 16-byte aligned data whose byte size is a multiple of 16 "
                         "(got %d bytes at offset %d)" % (b.numel(), b.data_ptr() % 16))

    def reduce_from_neighbours(self, t: torch.Tensor) -> torch.Tensor:
        """t <- t + left + right on a ring (communication.py:108-119); with two ranks the one peer counts twice."""
        if self.world == 1:
            return t
        dst, src, slot = self.plan.neighbours()
        b = _flat(t)
        if self.world == 2:
            other = torch.empty_like(t)
            self._exchange(dst, src, b, _flat(other), b.numel())
            return t.add_(other).add_(other)
        if b.numel() % 16 or b.data_ptr() % 16:
            self._reject(b)
        self._exchange(dst, src, b, b, b.numel(), reduce=_reduce_code(t), self_slot=slot)
        return t

    # ---- status ----------------------------------------------------------------------------------------------------
    def _state(self):
        st, src = C.c_uint32(0), C.c_int32(-1)
        N.check_cuda(_lib().esgd_coll_state(self.desc.data_ptr(), C.byref(st), C.byref(src), _stream()), "collective state")
        return int(st.value), int(src.value)

    def check(self) -> None:
        st, _ = self._state()
        if st:
            raise CollectiveError("; ".join(v for k, v in _STATUS.items() if st & k))

    def close(self) -> None:
        if self.arena is not None:
            torch.cuda.synchronize(self.device)
            self.arena.free()
            self.arena = None


class EmulatedCollectives:
    """``world`` ranks on ONE GPU.  Each method takes one tensor per rank and performs the collective for all of
    them with a single cooperative launch (one block per rank) over the device code of ``PeerCollectives``."""

    def __init__(self, world: int, device: torch.device, stage_kb: int = 256, timeout_s: float = 5.0):
        lib = _lib()
        self.world, self.device = world, device
        self.stage_bytes = _align(stage_kb << 10, 256)
        self.stage_off = _align(int(lib.esgd_coll_ctl_bytes()), 256)
        self.arenas = [torch.zeros(self.stage_off + self.stage_bytes, dtype=torch.uint8, device=device)
                       for _ in range(world)]
        nb = int(lib.esgd_coll_rank_bytes())
        self.descs = [torch.zeros(nb, dtype=torch.uint8, device=device) for _ in range(world)]
        bases = (C.c_uint64 * world)(*[a.data_ptr() for a in self.arenas])
        for r in range(world):
            N.check_cuda(lib.esgd_coll_init(self.descs[r].data_ptr(), r, world, bases, self.stage_off, timeout_s,
                                            _stream()), "collective descriptor")
        self.desc_ptrs = torch.tensor([d.data_ptr() for d in self.descs], dtype=torch.int64, device=device)
        self.plans = [_Plan(r, world) for r in range(world)]
        self.op_bytes = int(lib.esgd_coll_op_bytes())

    def _run(self, ops: Sequence[tuple]) -> None:
        """ops[r] = (dst_mask, src_mask, nbytes, in_ptr, out_ptr, out_stride, reduce, self_slot[, class])"""
        lib = _lib()
        host = (C.c_ubyte * (self.op_bytes * self.world))()
        for r, o in enumerate(ops):
            if o[2] > self.stage_bytes:
                raise ValueError("message larger than the emulated stage")
            lib.esgd_coll_pack_op(C.byref(host, r * self.op_bytes), *(tuple(o) + (COLLECTIVE,))[:9])
        dev = torch.frombuffer(bytearray(host), dtype=torch.uint8).to(self.device)
        N.check_cuda(lib.esgd_coll_exchange_emulated(self.desc_ptrs.data_ptr(), dev.data_ptr(), self.world, _stream()),
                     "emulated collective")
        torch.cuda.synchronize(self.device)

    def bcast(self, ts: List[torch.Tensor], root: int) -> None:
        ops = []
        for r, t in enumerate(ts):
            b = _flat(t)
            dst, src, _ = self.plans[r].bcast(root)
            ops.append((dst, src, b.numel(), b.data_ptr(), b.data_ptr(), 0, RED_NONE, -1))
        self._run(ops)

    def allgather(self, ts: List[torch.Tensor]) -> List[torch.Tensor]:
        outs = [torch.empty((self.world,) + tuple(t.shape), dtype=t.dtype, device=t.device) for t in ts]
        ops = []
        for r, t in enumerate(ts):
            b = _flat(t)
            dst, src, slot = self.plans[r].allgather()
            ops.append((dst, src, b.numel(), b.data_ptr(), outs[r].data_ptr(), b.numel(), RED_NONE, slot))
        self._run(ops)
        return outs

    def gather(self, ts: List[torch.Tensor], root: int) -> torch.Tensor:
        out = torch.empty((self.world,) + tuple(ts[0].shape), dtype=ts[0].dtype, device=ts[0].device)
        ops = []
        for r, t in enumerate(ts):
            b = _flat(t)
            dst, src, slot = self.plans[r].gather(root)
            ops.append((dst, src, b.numel(), b.data_ptr(), out.data_ptr() if r == root else 0, b.numel(), RED_NONE, slot))
        self._run(ops)
        return out

    def allreduce(self, ts: List[torch.Tensor]) -> None:
        ops = []
        for r, t in enumerate(ts):
            b = _flat(t)
            p = self.plans[r]
            ops.append((p.others, p.others, b.numel(), b.data_ptr(), b.data_ptr(), 0, _reduce_code(t), r))
        self._run(ops)

    def send_recv(self, t_src: torch.Tensor, src: int, t_dst: torch.Tensor, dst: int) -> None:
        ops = [(0, 0, 0, 0, 0, 0, RED_NONE, -1)] * self.world
        a, b = _flat(t_src), _flat(t_dst)
        ops[src] = (1 << dst, 0, a.numel(), a.data_ptr(), 0, 0, RED_NONE, -1, POINT_TO_POINT)
        ops[dst] = (0, 1 << src, b.numel(), 0, b.data_ptr(), 0, RED_NONE, -1, POINT_TO_POINT)
        self._run(ops)

    def neighbours(self, ts: List[torch.Tensor]) -> None:
        if self.world < 3:
            raise ValueError("the emulated ring sum needs three ranks or more")
        ops = []
        for r, t in enumerate(ts):
            b = _flat(t)
            dst, src, slot = self.plans[r].neighbours()
            ops.append((dst, src, b.numel(), b.data_ptr(), b.data_ptr(), 0, _reduce_code(t), slot))
        self._run(ops)

    def barrier(self) -> None:
        self._run([(p.others, p.others, 0, 0, 0, 0, RED_NONE, -1) for p in self.plans])

    def status(self) -> List[int]:
        out = []
        for d in self.descs:
            st, src = C.c_uint32(0), C.c_int32(-1)
            N.check_cuda(_lib().esgd_coll_state(d.data_ptr(), C.byref(st), C.byref(src), _stream()), "collective state")
            out.append(int(st.value))
        return out
