"""Process group: rank/size, bootstrap exchange and the classic collectives.

Counterpart of the reference's ``CommunicationNetwork``
(deep500/lv3/communication.py:14-119: size, rank, sync_all, gather_at_root,
sync_all_with_root, send_to_root, wait_for_any_rank, send_to_rank,
wait_for_root, reduce_from_neighbors) and of ffinit/ffrank/ffsize
(fflib2 src/ff.h:100-104).  On GPUs the data collectives are this package's own
kernels over peer memory (``parallel/peer_collectives.py``); ``torch.distributed`` is the
bootstrap plane (gloo object exchange, barrier) and the CPU path.  One process per GPU.
"""
from __future__ import annotations

import os
from typing import Any, List, Optional

import torch
import torch.distributed as dist

_default_group: Optional["Group"] = None


class Group:
    def __init__(self, backend: Optional[str] = None, device: Optional[torch.device] = None):
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", str(self.rank)))
        if device is None:
            use_cuda = torch.cuda.is_available() and backend != "gloo"
            device = torch.device("cuda", self.local_rank) if use_cuda else torch.device("cpu")
        self.device = device
        if device.type == "cuda":
            torch.cuda.set_device(device)
        self.backend = backend or ("nccl" if device.type == "cuda" else "gloo")
        self._own_pg = False
        self.gloo = None
        self._peer = None
        if self.world > 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29511")
            if not dist.is_initialized():
                kwargs = {}
                if self.backend == "nccl":
                    kwargs["device_id"] = device
                dist.init_process_group(self.backend, rank=self.rank, world_size=self.world, **kwargs)
                self._own_pg = True
            # object exchange (IPC handles, shm names) never needs the GPU
            self.gloo = dist.new_group(backend="gloo") if self.backend != "gloo" else dist.group.WORLD

    # ---- identity (ffrank / ffsize) -------------------------------------
    @property
    def size(self) -> int:
        return self.world

    def is_root(self) -> bool:
        return self.rank == 0

    # ---- bootstrap ---------------------------------------------------------
    def exchange(self, obj: Any) -> List[Any]:
        """All-gather a small python object (used for IPC handles and shm names)."""
        if self.world == 1:
            return [obj]
        out: List[Any] = [None] * self.world
        dist.all_gather_object(out, obj, group=self.gloo)
        return out

    # ---- this package's own collectives over peer memory ------------------------------------------------
    def peer_collectives(self, stage_mb: float = 64.0):
        """The kernels of ``parallel/peer_collectives.py`` for this group (created on first use; every rank must
        make that first call at the same point, since the arenas are exchanged then)."""
        if self._peer is None:
            from .peer_collectives import PeerCollectives
            self._peer = PeerCollectives(self.rank, self.world, self.exchange, stage_mb=stage_mb, device=self.device)
        return self._peer

    def _native(self, t: torch.Tensor, summed: bool = False) -> bool:
        """Whether a collective on ``t`` runs on this package's kernels: CUDA tensors of a multi-rank group, unless
        ``ESGD_NATIVE_COLLECTIVES=0``; sums only for float32 / bfloat16 in 16-byte units."""
        if self.world == 1 or not t.is_cuda or not t.is_contiguous() or os.environ.get("ESGD_NATIVE_COLLECTIVES", "1") == "0":
            return False
        if summed and (t.dtype not in (torch.float32, torch.bfloat16) or (t.numel() * t.element_size()) % 16
                       or t.data_ptr() % 16):
            return False
        return True

    def barrier(self) -> None:
        if self.world > 1:
            if self.backend == "nccl":
                dist.barrier(device_ids=[self.device.index])
            else:
                dist.barrier()

    # ---- CommunicationNetwork parity --------------------------------------
    def sync_all(self, t: torch.Tensor, average: bool = False) -> torch.Tensor:
        """In-place allreduce-sum over every rank (``sync_all``, communication.py:88-98)."""
        if self._native(t, summed=True):
            self.peer_collectives().allreduce(t)
        elif self.world > 1:
            dist.all_reduce(t)
        if average:
            t.div_(self.world)
        return t

    allreduce = sync_all

    def sync_all_at_root(self, t: torch.Tensor, average: bool = False) -> torch.Tensor:
        """Sum over every rank, delivered to rank 0 only (``sync_all_at_root``, communication.py: a reduce);
        the other ranks' tensors are left as they are."""
        if self.world == 1:
            return t.div_(1) if average else t
        if self._native(t):
            parts = self.peer_collectives().gather(t, 0)
            if parts is not None:
                t.copy_(parts.sum(0) if t.is_floating_point() else parts.sum(0).to(t.dtype))
        else:
            dist.reduce(t, dst=0)
        if average and self.rank == 0:
            t.div_(self.world)
        return t

    def gather_at_root(self, t: torch.Tensor) -> Optional[List[torch.Tensor]]:
        if self.world == 1:
            return [t.clone()]
        if self._native(t):
            out = self.peer_collectives().gather(t, 0)
            return list(out.unbind(0)) if out is not None else None
        out = [torch.empty_like(t) for _ in range(self.world)]
        dist.all_gather(out, t)  # gather() is not available on every backend
        return out if self.rank == 0 else None

    def sync_all_with_root(self, t: torch.Tensor, root: int = 0) -> torch.Tensor:
        if self._native(t):
            self.peer_collectives().bcast(t, root)
        elif self.world > 1:
            dist.broadcast(t, src=root)
        return t

    bcast = sync_all_with_root

    def send_to_rank(self, t: torch.Tensor, dst: int, tag: int = 0) -> None:
        if self._native(t):
            return self.peer_collectives().send(t, dst)   # matched by order per pair of ranks; the tag is not needed
        dist.send(t, dst=dst, tag=tag)

    def send_to_root(self, t: torch.Tensor, tag: int = 0) -> None:
        self.send_to_rank(t, 0, tag)

    def wait_for_rank(self, t: torch.Tensor, src: int, tag: int = 0) -> int:
        if self._native(t):
            return self.peer_collectives().recv(t, src)
        dist.recv(t, src=src, tag=tag)
        return src

    def wait_for_root(self, t: torch.Tensor, tag: int = 0) -> int:
        return self.wait_for_rank(t, 0, tag)

    def wait_for_any_rank(self, t: torch.Tensor, tag: int = 0) -> int:
        """Receive from whichever rank sends first; returns the source rank."""
        if self._native(t):
            return self.peer_collectives().recv_any(t)
        return dist.recv(t, src=None, tag=tag)

    def reduce_from_neighbors(self, t: torch.Tensor) -> torch.Tensor:
        """t <- t + left + right on a ring (``reduce_from_neighbors``, communication.py:108-119)."""
        if self.world == 1:
            return t
        if self._native(t, summed=True):
            return self.peer_collectives().reduce_from_neighbours(t)
        left, right = (self.rank - 1) % self.world, (self.rank + 1) % self.world
        if self.world == 2:
            other = torch.empty_like(t)
            ops = [dist.P2POp(dist.isend, t.clone(), left), dist.P2POp(dist.irecv, other, left)]
            for r in dist.batch_isend_irecv(ops):
                r.wait()
            return t.add_(other).add_(other)
        from_left, from_right = torch.empty_like(t), torch.empty_like(t)
        snd = t.clone()
        ops = [dist.P2POp(dist.isend, snd, left), dist.P2POp(dist.isend, snd, right),
               dist.P2POp(dist.irecv, from_left, left), dist.P2POp(dist.irecv, from_right, right)]
        for r in dist.batch_isend_irecv(ops):
            r.wait()
        return t.add_(from_left).add_(from_right)

    def finalize(self) -> None:
        if self._peer is not None:
            self._peer.close()
            self._peer = None
        if self._own_pg and dist.is_initialized():
            dist.destroy_process_group()
            self._own_pg = False


def init(backend: Optional[str] = None, device: Optional[torch.device] = None) -> Group:
    """Create (or return) the default group (``ffinit``, fflib2 src/ff.c:23-86)."""
    global _default_group
    if _default_group is None:
        _default_group = Group(backend, device)
    return _default_group


def finalize() -> None:
    global _default_group
    if _default_group is not None:
        _default_group.finalize()
        _default_group = None


def rank() -> int:
    return init().rank


def world_size() -> int:
    return init().world
