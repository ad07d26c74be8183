"""Partial-allreduce micro-benchmark: solo vs majority vs synchronous (ours) vs NCCL allreduce.

    torchrun --nproc-per-node 8 -m eagersgd_b200.parallel.bench_allreduce --sizes 4096,1048576,268435456 --late 2

For every buffer size and dtype, ``--iters`` rounds are timed on the device: all ranks are aligned
with a barrier, every rank holds its stream for ``--hold-us`` with a bounded spin kernel (so that the
launches that follow are already queued when the clock starts and host launch overhead is not part of
the figure), ``--late`` seeded-random ranks hold it longer by U(0, ``--late-ms``), and each rank measures
the time from its own arrival to the completion of its collective (CUDA events).  Reported per case: mean and max over ranks of the per-rank latency
(the reference's SGD-loop tests print the mean over ranks: fflib2 evaluation/ssgd.c:75-95, rsgd.c:
90-111, randomsgd.c:90-111) and, for the synchronous variants, the bus bandwidth
2(P-1)/P * bytes / time.  Same protocol as the reference's allreduce micro-benchmark
(fflib2 benchmark/allreduce.c: fixed iteration count, library vs MPI_Allreduce) with NCCL in the
role of MPI_Allreduce.  Rank 0 prints one JSON line per case.
"""
from __future__ import annotations

import argparse
import json
import random
import sys

import torch
import torch.distributed as dist

from . import _native as N
from .group import init as init_group, finalize
from .nvlink_channel import NvlinkChannel, TWO_SHOT_MIN, create_arenas


def run_case(group, nbytes, dtype, mode, late, late_ms, iters, seed, fused, one_shot=False, grace_us=50.0,
             hold_us=300.0, multicast=True, zero_copy=False):
    dev = group.device
    esz = 2 if dtype == torch.bfloat16 else 4
    count = max(nbytes // esz // 8 * 8, 8)
    grad = torch.randn(count, device=dev).to(dtype)
    stream = torch.cuda.current_stream(dev)
    rng = random.Random(seed)
    ch = arena = None
    if mode != "nccl":
        arena, bases = create_arenas(count, dtype, group.rank, group.world, group.exchange,
                                     multicast=None if multicast else False)
        kw = {}
        if fused:
            kw = dict(w32=torch.zeros(count, device=dev), mom=torch.zeros(count, device=dev),
                      w16=torch.zeros(count, dtype=torch.bfloat16, device=dev) if dtype == torch.bfloat16 else None)
        else:
            kw = dict(out=torch.empty(count, dtype=dtype, device=dev))
        ch = NvlinkChannel(count, group.rank, group.world, bases, dev, None if zero_copy else grad, slot_dtype=dtype,
                           mode=mode, limiter=-1,
                           average="world", timeout_s=20.0, grace_us=grace_us,
                           two_shot_min=None if one_shot else TWO_SHOT_MIN, mc_base=arena.mc_base, **kw)
    buf = grad.clone()
    times, phases = [], {}
    for it in range(iters + 3):
        delays = [0.0] * group.world
        for _ in range(late):
            delays[rng.randrange(group.world)] = rng.uniform(0, late_ms * 1e-3)
        if ch is not None and zero_copy:
            ch.publish_view().copy_(grad)      # outside the timed region, like filling NCCL's buffer
        group.barrier()
        hold_ns = int(hold_us * 1e3 + delays[group.rank] * 1e9)
        if hold_ns > 0:
            N.check_cuda(N.cuda().esgd_spin(hold_ns, stream.cuda_stream), "delay")
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        if mode == "nccl":
            dist.all_reduce(buf)
            buf.div_(group.world)
        else:
            ch.step()
        e1.record()
        torch.cuda.synchronize()
        if it >= 3:
            times.append(e0.elapsed_time(e1))
            if ch is not None:
                for kk, vv in ch.phase_times_us().items():
                    if vv is not None:
                        phases.setdefault(kk, []).append(vv)
    t = torch.tensor([sum(times) / len(times)], device=dev)
    tmax, tsum = t.clone(), t.clone()
    if group.world > 1:
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        dist.all_reduce(tsum)
    status, control_us = 0, None
    if ch is not None:
        ch.flush()
        torch.cuda.synchronize()
        st = ch.stats()
        status, control_us = st["status"], st.get("control_us")
        group.barrier()
        arena.free()
    mean_ms, max_ms = float(tsum) / group.world, float(tmax)
    res = dict(mode=mode, bytes=count * esz, dtype=str(dtype).replace("torch.", ""), world=group.world, late=late,
               late_ms=late_ms, fused_update=bool(fused and mode != "nccl"), mean_latency_us=mean_ms * 1e3,
               max_latency_us=max_ms * 1e3, status=status,
               two_shot=bool(ch is not None and ch.two_shot), multicast=bool(ch is not None and ch.multicast),
               zero_copy=bool(zero_copy and ch is not None))
    if control_us is not None:
        res["control_us_last"] = control_us
    if phases:   # this rank's device-side break-down of its steps
        res["phases_us"] = {kk: round(sum(vv) / len(vv), 1) for kk, vv in phases.items()}
    if mode in ("sync", "nccl") and late == 0:
        res["bus_gbs"] = 2.0 * (group.world - 1) / max(group.world, 1) * count * esz / (max_ms * 1e-3) / 1e9
    return res


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes", default="4096,65536,1048576,16777216,268435456")
    ap.add_argument("--dtypes", default="float32,bfloat16")
    ap.add_argument("--modes", default="solo,majority,sync,nccl")
    ap.add_argument("--late", type=int, default=0, help="ranks arriving late each round")
    ap.add_argument("--late-ms", type=float, default=10.0)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--fused", action="store_true", help="include the fused momentum-SGD update in our kernels")
    ap.add_argument("--one-shot", action="store_true", help="never split the reduction into reduce-scatter + gather")
    ap.add_argument("--zero-copy", action="store_true",
                    help="write the gradient straight into the publish slot (no staging copy inside the timed step)")
    ap.add_argument("--no-multicast", action="store_true",
                    help="plain peer loads only: no in-switch (multimem) reduction of rounds in which all are on time")
    ap.add_argument("--grace-us", type=float, default=50.0,
                    help="longest time an activator waits for near-simultaneous arrivals (the window adapts below it)")
    ap.add_argument("--hold-us", type=float, default=300.0,
                    help="every rank holds its stream this long before the timed region, so the launches are queued")
    args = ap.parse_args(argv)
    group = init_group()
    for size in [int(s) for s in args.sizes.split(",")]:
        for dt in args.dtypes.split(","):
            for mode in args.modes.split(","):
                r = run_case(group, size, getattr(torch, dt), mode, args.late, args.late_ms, args.iters, 1234, args.fused,
                             args.one_shot, args.grace_us, args.hold_us, not args.no_multicast,
                             args.zero_copy)
                if group.rank == 0:
                    print(json.dumps(r), flush=True)
    finalize()
    return 0


if __name__ == "__main__":
    sys.exit(main())
