"""CPU backend of the partial allreduce (ranks = threads or processes of one host).

The control protocol is the very code the CUDA kernels run, instantiated with
host atomics over shared memory (``csrc/host/cpu_channel.cpp``).  It stands in
for the reference's host path, fflib2 over MPI (src/colls/ffsolo_allreduce.c,
ffrand_allreduce.c, ffallreduce.c), which is how eager-SGD runs without a GPU.
"""
from __future__ import annotations

import atexit
import ctypes as C
import os
import uuid
from multiprocessing import shared_memory
from typing import List, Optional, Sequence

import numpy as np
import torch

from . import _native as N

_NP_DTYPES = {np.dtype("float32"): N.DT_F32, np.dtype("float64"): N.DT_F64,
              np.dtype("int32"): N.DT_I32, np.dtype("int64"): N.DT_I64}
_MODES = {"solo": N.MODE_SOLO, "majority": N.MODE_MAJORITY, "sync": N.MODE_SYNC}
_AVG = {"contributors": N.AVG_CONTRIBUTORS, "world": N.AVG_WORLD, "sum": N.AVG_SUM}


def segment_bytes(count: int, np_dtype) -> int:
    return int(N.host().esgd_cpu_segment_bytes(count, _NP_DTYPES[np.dtype(np_dtype)]))


class LocalSegments:
    """Segments of every rank inside one process (ranks are threads)."""

    def __init__(self, world: int, count: int, np_dtype):
        nbytes = segment_bytes(count, np_dtype)
        self._raw = [np.zeros(nbytes + 256, dtype=np.uint8) for _ in range(world)]
        self.bases = [a.ctypes.data + ((-a.ctypes.data) % 256) for a in self._raw]

    def close(self):
        self._raw = []


class SharedSegments:
    """One POSIX shared-memory segment per rank, opened by every process of the group.

    ``exchange`` is a callable that all-gathers a python object over the group
    (``torch.distributed.all_gather_object`` on a gloo group, typically).
    """

    def __init__(self, rank: int, world: int, count: int, np_dtype, exchange):
        nbytes = segment_bytes(count, np_dtype)
        self.rank = rank
        name = "esgd_%d_%s" % (os.getpid(), uuid.uuid4().hex[:12])
        self._own = shared_memory.SharedMemory(name=name, create=True, size=nbytes)
        np.frombuffer(self._own.buf, dtype=np.uint8)[:] = 0
        names = exchange(name)
        self._peers: List[Optional[shared_memory.SharedMemory]] = []
        for r, nm in enumerate(names):
            if r == rank:
                self._peers.append(None)
            else:
                seg = shared_memory.SharedMemory(name=nm, create=False)
                try:  # the creator unlinks; do not let this process's tracker do it too
                    from multiprocessing import resource_tracker
                    resource_tracker.unregister(seg._name, "shared_memory")
                except Exception:
                    pass
                self._peers.append(seg)
        self._views = []
        self.bases = []
        for r in range(world):
            seg = self._own if r == rank else self._peers[r]
            view = np.frombuffer(seg.buf, dtype=np.uint8)
            self._views.append(view)
            self.bases.append(view.ctypes.data)
        exchange("ready")  # every peer has mapped every segment before anyone proceeds
        self._closed = False
        atexit.register(self.close)   # a program that forgets close() still unmaps and unlinks in the right order

    def close(self):
        if getattr(self, "_closed", True):
            return
        self._closed = True
        self._views = []
        self.bases = []
        for seg in self._peers:
            if seg is not None:
                try:
                    seg.close()
                except BufferError:
                    pass
        try:
            self._own.close()
        except BufferError:
            pass
        try:
            # ranks started by one parent share its resource tracker, and a peer's unregister (above) has then
            # removed this segment's entry as well: put it back so that unlink() finds what it takes out
            from multiprocessing import resource_tracker
            resource_tracker.register(self._own._name, "shared_memory")
        except Exception:
            pass
        try:
            self._own.unlink()
        except FileNotFoundError:
            pass


class CpuChannel:
    """A persistent partial allreduce over ``count`` elements on the CPU."""

    def __init__(self, bases: Sequence[int], rank: int, world: int, count: int, np_dtype=np.float32,
                 mode: str = "solo", limiter: int = 32, seed: int = 6545343, average: str = "contributors",
                 include_stale: bool = True, timeout_s: float = 60.0, grace_us: float = 0.0, home: int = 0,
                 accumulate: bool = False, adaptive_grace: bool = False):
        self.lib = N.host()
        self.rank, self.world, self.count = rank, world, count
        self.np_dtype = np.dtype(np_dtype)
        if self.np_dtype.kind == "i" and average != "sum":
            raise ValueError("integer buffers support average='sum' only")
        self._bases = (C.c_void_p * world)(*bases)
        self.params = N.CpuParams(rank=rank, world=world, base_mode=_MODES[mode], include_stale=int(include_stale),
                                  average=_AVG[average], home=home, dtype=_NP_DTYPES[self.np_dtype],
                                  flags=int(accumulate) | (int(adaptive_grace) << 1),
                                  limiter=limiter, seed=seed, timeout_ns=int(timeout_s * 1e9),
                                  grace_ns=int(grace_us * 1e3), count=count)
        self.info = N.StepInfo()

    def _as_np(self, t):
        if isinstance(t, torch.Tensor):
            t = t.detach().contiguous().numpy()
        a = np.ascontiguousarray(t, dtype=self.np_dtype).reshape(-1)
        if a.size != self.count:
            raise ValueError("expected %d elements, got %d" % (self.count, a.size))
        return a

    def step(self, grad, out: Optional[np.ndarray] = None):
        """Publish ``grad``, take part in or absorb one round; returns (gradient to apply, info)."""
        g = self._as_np(grad)
        if out is None:
            out = np.empty(self.count, dtype=self.np_dtype)
        st = self.lib.esgd_cpu_step(self._bases, C.byref(self.params), g.ctypes.data, out.ctypes.data,
                                    C.byref(self.info))
        if st != 0:
            raise N.ChannelError(st, "cpu rank %d step %d" % (self.rank, self.info.local_step))
        return out, self.info

    def flush(self, out: Optional[np.ndarray] = None):
        if out is None:
            out = np.empty(self.count, dtype=self.np_dtype)
        st = self.lib.esgd_cpu_flush(self._bases, C.byref(self.params), out.ctypes.data, C.byref(self.info))
        if st != 0:
            raise N.ChannelError(st, "cpu rank %d flush" % self.rank)
        return out, self.info

    def trace(self) -> list:
        return N.parse_trace(C.c_void_p(self._bases[self.rank]))

    def stats(self) -> dict:
        raw = (C.c_uint64 * 24)()
        self.lib.esgd_ctl_stats(C.c_void_p(self._bases[self.rank]), raw)
        return N.parse_stats(raw)
