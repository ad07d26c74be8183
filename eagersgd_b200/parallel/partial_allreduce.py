"""``PartialAllreduce``: one persistent partial allreduce over one tensor, with the life cycle of the reference's
schedules — create once, ``start``, then ``post`` / ``wait`` (or ``test``) every iteration, ``close`` at the end.

It stands where a user of the reference calls ``ffsolo_allreduce`` / ``ffrand_allreduce`` / ``ffallreduce`` and drives
the returned schedule with ``ffschedule_{start,post,wait,test,delete,print}`` (fflib2 src/ff.h:137-165,
src/colls/ffsolo_allreduce.c:88-148, evaluation/rsgd.c:77-113).  Here the object picks the backend from the tensor:
a CUDA tensor runs on the NVLink kernels (``post`` launches them on a side stream and returns, ``wait`` joins the
stream), a CPU tensor on the shared-memory channel (``post`` hands the step to a worker thread, like the reference's
progress thread, and returns).  The optimizer wrappers use the same channels bucket by bucket; this class is for
programs that want the collective by itself.

    ar = PartialAllreduce(grad, group, mode="solo", limiter=32)      # result written back into ``grad``
    ar.start()
    for _ in range(steps):
        fill(grad)
        ar.post()
        ...                       # overlap something
        info = ar.wait()          # info["role"], info["contributors"], ...
    ar.close()
"""
from __future__ import annotations

import threading
from typing import Callable, Optional

import numpy as np
import torch

from . import _native as N
from .group import Group

_ROLES = {N.ROLE_PARTICIPANT: "participant", N.ROLE_DRAIN: "drain"}      # anything else: the rank missed the round


class PartialAllreduce:
    def __init__(self, tensor: torch.Tensor, group: Group, mode: str = "solo", limiter: int = 32, seed: int = 6545343,
                 average: str = "contributors", out: Optional[torch.Tensor] = None, accumulate: bool = False,
                 timeout_s: float = 60.0, grace_us: float = 50.0, on_complete: Optional[Callable[[dict], None]] = None):
        """``tensor``: flat or shaped, contiguous; its element count is fixed for the life of the object (use
        ``resize`` for another).  ``out``: where the averaged result goes (default: in place).  ``mode``: "solo",
        "majority" or "sync"; ``limiter``: eager rounds between two forced synchronous ones (solo / majority);
        ``average``: "contributors" (divide by how many gradients a round summed), "world" (the reference's behaviour)
        or "sum".  ``on_complete(info)`` runs when a posted round has completed (inside ``wait`` / a successful
        ``test``)."""
        if not tensor.is_contiguous() or (out is not None and (not out.is_contiguous() or out.shape != tensor.shape)):
            raise ValueError("PartialAllreduce takes contiguous tensors of one shape")
        self.group, self.mode, self.limiter, self.seed, self.average = group, mode, limiter, seed, average
        self.accumulate, self.timeout_s, self.grace_us, self.on_complete = accumulate, timeout_s, grace_us, on_complete
        self._kw = dict(mode=mode, limiter=limiter if mode != "sync" else -1, seed=seed, average=average,
                        timeout_s=timeout_s, accumulate=accumulate)
        self._started = self._posted = False
        self._last: dict = {}
        self._bind(tensor, out)

    # ---- construction --------------------------------------------------------------------------------------------
    def _bind(self, tensor: torch.Tensor, out: Optional[torch.Tensor]) -> None:
        g = self.group
        self.tensor, self.out = tensor, out if out is not None else tensor
        n = tensor.numel()
        self.count = (n + 7) // 8 * 8                       # the kernels work in units of eight elements
        self.on_gpu = tensor.is_cuda
        if self.on_gpu:
            from .nvlink_channel import NvlinkChannel, create_arenas
            if tensor.dtype not in (torch.float32, torch.bfloat16):
                raise ValueError("GPU tensors must be float32 or bfloat16")
            dev = tensor.device
            self._grad = tensor.view(-1) if n == self.count else torch.zeros(self.count, dtype=tensor.dtype, device=dev)
            self._res = (self.out.view(-1) if n == self.count else torch.zeros(self.count, dtype=torch.float32, device=dev))
            if self._res.dtype != torch.float32:           # the kernels write fp32 averages (or bf16 working copies)
                self._res = torch.zeros(self.count, dtype=torch.float32, device=dev)
            self._arena, bases = create_arenas(self.count, tensor.dtype, g.rank, g.world, g.exchange)
            self._stream = torch.cuda.Stream(device=dev)
            self._done = torch.cuda.Event()
            self._ch = NvlinkChannel(self.count, g.rank, g.world, bases, dev, self._grad, slot_dtype=tensor.dtype,
                                     out=self._res, grace_us=self.grace_us, mc_base=self._arena.mc_base, **self._kw)
        else:
            from .cpu_channel import CpuChannel, LocalSegments, SharedSegments
            npdt = {torch.float32: np.float32, torch.float64: np.float64, torch.int32: np.int32,
                    torch.int64: np.int64}.get(tensor.dtype)
            if npdt is None:
                raise ValueError("CPU tensors must be float32, float64, int32 or int64")
            self.count = n
            self._seg = (LocalSegments(1, n, npdt) if g.world == 1 else SharedSegments(g.rank, g.world, n, npdt, g.exchange))
            self._ch = CpuChannel(self._seg.bases, g.rank, g.world, n, npdt, grace_us=0.0, **self._kw)
            self._np_out = np.empty(n, dtype=npdt)
            self._thread: Optional[threading.Thread] = None
            self._err: Optional[BaseException] = None
        g.barrier()                                          # every rank's channel exists before anybody posts

    # ---- life cycle (ffschedule_start / post / wait / test / delete) ---------------------------------------------
    def start(self) -> "PartialAllreduce":
        """Arm the collective (the reference posts its receives here; with one-sided peer memory there is nothing
        to arm, so this only marks the object as usable)."""
        self._started = True
        return self

    def post(self) -> None:
        """Publish the tensor's current content and take part in (or miss) a round; returns at once."""
        if not self._started:
            raise RuntimeError("start() the collective before posting")
        if self._posted:
            raise RuntimeError("the previous post has not been waited for")
        if self.on_gpu:
            cur = torch.cuda.current_stream(self.tensor.device)
            if self._grad.data_ptr() != self.tensor.data_ptr():
                self._grad[:self.tensor.numel()].copy_(self.tensor.view(-1))
            self._stream.wait_stream(cur)
            self._ch.step(self._stream)
            self._done.record(self._stream)
        else:
            src = self.tensor.detach().view(-1).numpy().copy()

            def run():
                try:
                    self._ch.step(src, self._np_out)
                except BaseException as e:  # noqa: reported by wait()
                    self._err = e

            self._thread = threading.Thread(target=run, daemon=True)
            self._thread.start()
        self._posted = True

    def test(self) -> bool:
        """Has the posted round completed?  Completes it (like ``wait``) when it has."""
        if not self._posted:
            return True
        done = self._done.query() if self.on_gpu else not self._thread.is_alive()
        if done:
            self.wait()
        return done

    def wait(self) -> dict:
        """Block until the posted round has completed on this rank; the result is then in ``out`` (or in place).
        Returns what happened: role, round, contributors, whether the round was a synchronous one."""
        if not self._posted:
            return self._last
        if self.on_gpu:
            torch.cuda.current_stream(self.tensor.device).wait_stream(self._stream)
            self._done.synchronize()
            self._ch.check("partial allreduce")
            n = self.tensor.numel()
            if self._ch.applied():
                if self._res.data_ptr() != self.out.data_ptr():
                    self.out.view(-1).copy_(self._res[:n])
            tr = self._ch.trace()
            last = tr[-1] if tr else {}
            role = last.get("role")
            info = {"role": role if role in ("participant", "drain") else "absent", "round": last.get("round"),
                    "contributors": bin(int(last.get("contrib_mask", 0))).count("1"), "sync": bool(last.get("is_sync", 0)),
                    "applied": self._ch.applied()}
        else:
            self._thread.join()
            self._thread = None
            if self._err is not None:
                e, self._err = self._err, None
                self._posted = False
                raise e
            i = self._ch.info
            applied = i.role in (N.ROLE_PARTICIPANT, N.ROLE_DRAIN)
            if applied:
                self.out.view(-1).copy_(torch.from_numpy(self._np_out))
            info = {"role": _ROLES.get(i.role, "absent"), "round": int(i.round), "contributors": int(i.n_contrib),
                    "sync": bool(i.is_sync), "applied": applied}
        self._posted = False
        self._last = info
        if self.on_complete is not None:
            self.on_complete(info)
        return info

    def flush(self) -> dict:
        """Collect what rounds this rank missed have left for it (call once after the last step)."""
        if self._posted:
            self.wait()
        if self.on_gpu:
            self._ch.flush(self._stream)
            self._stream.synchronize()
            if self._ch.applied() and self._res.data_ptr() != self.out.data_ptr():
                self.out.view(-1).copy_(self._res[:self.tensor.numel()])
        else:
            out, i = self._ch.flush(self._np_out)
            if i.role in (N.ROLE_PARTICIPANT, N.ROLE_DRAIN):
                self.out.view(-1).copy_(torch.from_numpy(out))
        return self.stats()

    def resize(self, tensor: torch.Tensor, out: Optional[torch.Tensor] = None) -> None:
        """Continue with a tensor of another size (the reference's ``ffbuffer_resize`` between posts): every rank
        must call this at the same point; the channel is rebuilt."""
        self._release()
        self._bind(tensor, out)

    def describe(self) -> str:
        """One paragraph on what this object is (the counterpart of ``ffschedule_print``)."""
        s = self.stats()
        return ("partial allreduce [%s] of %d x %s on %s, rank %d of %d, limiter %s, average by %s; steps %d, took part in %d,"
                " missed %d, forced synchronous rounds %d" %
                (self.mode, self.tensor.numel(), str(self.tensor.dtype).replace("torch.", ""),
                 "NVLink peer memory" if self.on_gpu else "shared memory", self.group.rank, self.group.world,
                 self.limiter if self.mode != "sync" else "-", self.average, s["steps"], s["participated"], s["absent"],
                 s["forced_sync"]))

    def stats(self) -> dict:
        """Counters of this rank: steps, participated, absent, activated, forced_sync (rounds the limiter or the
        mode made synchronous), dropped_grads, folded_grads, mean_contributors, wait_ms, status."""
        r = self._ch.stats()
        return {"steps": r["local_step"], "participated": r["participated"], "absent": r["absent"],
                "activated": r["activated"], "forced_sync": r["sync_rounds"], "dropped_grads": r["dropped_grads"],
                "folded_grads": r["folded_grads"], "wait_ms": r["wait_ns"] / 1e6, "status": r["status"],
                "mean_contributors": r["contrib_sum"] / max(1, r["participated"])}

    def _release(self) -> None:
        if self._posted:
            self.wait()
        self.group.barrier()                                 # nobody frees memory a peer may still read
        if self.on_gpu:
            torch.cuda.synchronize(self.tensor.device)
            self._arena.free()
        else:
            self._seg.close()

    def close(self) -> None:
        """Release the channel (``ffschedule_delete``); every rank calls it at the same point."""
        if getattr(self, "_ch", None) is not None:
            self._release()
            self._ch = None

    def __enter__(self):
        return self.start()

    def __exit__(self, *exc):
        self.close()
        return False
