"""Process group: rank/size, bootstrap exchange and the classic collectives.

Counterpart of the reference's ``CommunicationNetwork``
(deep500/lv3/communication.py:14-119: size, rank, sync_all, gather_at_root,
sync_all_with_root, send_to_root, wait_for_any_rank, send_to_rank,
wait_for_root, reduce_from_neighbors) and of ffinit/ffrank/ffsize
(fflib2 src/ff.h:100-104), on ``torch.distributed`` (NCCL on GPUs for bulk
data, gloo for object exchange and CPU runs).  One process per GPU.
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

    def barrier(self) -> None:
        if self.world > 1:
            if self.backend == "nccl":
                dist.barrier(device_ids=[self.device.index])
            else:
                dist.barrier()

    # ---- CommunicationNetwork parity --------------------------------------
    def sync_all(self, t: torch.Tensor, average: bool = False) -> torch.Tensor:
        """In-place allreduce-sum over every rank (``sync_all``, communication.py:88-98)."""
        if self.world > 1:
            dist.all_reduce(t)
        if average:
            t.div_(self.world)
        return t

    allreduce = sync_all

    def gather_at_root(self, t: torch.Tensor) -> Optional[List[torch.Tensor]]:
        if self.world == 1:
            return [t.clone()]
        out = [torch.empty_like(t) for _ in range(self.world)]
        dist.all_gather(out, t)  # gather() is not available on every backend
        return out if self.rank == 0 else None

    def sync_all_with_root(self, t: torch.Tensor, root: int = 0) -> torch.Tensor:
        if self.world > 1:
            dist.broadcast(t, src=root)
        return t

    bcast = sync_all_with_root

    def send_to_rank(self, t: torch.Tensor, dst: int, tag: int = 0) -> None:
        dist.send(t, dst=dst, tag=tag)

    def send_to_root(self, t: torch.Tensor, tag: int = 0) -> None:
        self.send_to_rank(t, 0, tag)

    def wait_for_rank(self, t: torch.Tensor, src: int, tag: int = 0) -> int:
        dist.recv(t, src=src, tag=tag)
        return src

    def wait_for_root(self, t: torch.Tensor, tag: int = 0) -> int:
        return self.wait_for_rank(t, 0, tag)

    def wait_for_any_rank(self, t: torch.Tensor, tag: int = 0) -> int:
        """Receive from whichever rank sends first; returns the source rank."""
        return dist.recv(t, src=None, tag=tag)

    def reduce_from_neighbors(self, t: torch.Tensor) -> torch.Tensor:
        """t <- t + left + right on a ring (``reduce_from_neighbors``, communication.py:108-119)."""
        if self.world == 1:
            return t
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
