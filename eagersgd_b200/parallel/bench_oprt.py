"""Micro-benchmark of the host operation runtime: creation, execution and deletion of an allreduce schedule.

    python -m eagersgd_b200.parallel.bench_oprt [--ranks 4] [--count 1024] [--iters 100] [--python-threads]

The protocol of the reference's benchmark (fflib2 benchmark/allreduce.c:11-99: int32, 100 timed iterations,
schedule creation / execution / deletion recorded separately), with ranks as threads of this process and a
plain numpy sum over the ranks' buffers as the baseline where the reference uses ``MPI_Allreduce``.
Prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import sys
import threading
import time

import numpy as np

from . import oprt as R


def run(ranks: int, count: int, iters: int) -> dict:
    t_create = [0.0] * ranks
    t_exec = [0.0] * ranks
    ok = [True] * ranks
    with R.World(ranks) as w:
        barrier = threading.Barrier(ranks)

        def body(r):
            snd = np.zeros(count, dtype=np.int32)
            rcv = np.zeros(count, dtype=np.int32)
            t0 = time.perf_counter()
            s = r.allreduce(r.buffer(snd), r.buffer(rcv), tag=1)
            t_create[r.id] = time.perf_counter() - t0
            for it in range(iters + 5):
                snd[:] = r.id + it
                barrier.wait()
                t0 = time.perf_counter()
                r.schedule_post(s)
                r.schedule_wait(s)
                if it >= 5:
                    t_exec[r.id] += time.perf_counter() - t0
                ok[r.id] = ok[r.id] and bool(np.all(rcv == it * ranks + ranks * (ranks - 1) // 2))
        th = [threading.Thread(target=body, args=(w.ranks[i],)) for i in range(ranks)]
        t0 = time.perf_counter()
        [t.start() for t in th]
        [t.join() for t in th]
        t_total = time.perf_counter() - t0
        t0 = time.perf_counter()
    t_delete = time.perf_counter() - t0                       # world (and every schedule in it) torn down
    bufs = [np.full(count, i, dtype=np.int32) for i in range(ranks)]
    t0 = time.perf_counter()
    for _ in range(iters):
        np.sum(bufs, axis=0)
    t_numpy = (time.perf_counter() - t0) / iters
    return {"ranks": ranks, "count": count, "dtype": "int32", "iters": iters, "correct": all(ok),
            "create_us": 1e6 * max(t_create), "execute_us": 1e6 * max(t_exec) / iters, "delete_us": 1e6 * t_delete,
            "numpy_sum_us": 1e6 * t_numpy, "wall_s": t_total}


def run_native(ranks: int, count: int, iters: int) -> dict:
    """The same protocol with native threads as ranks (no interpreter in the loop): microseconds per post + wait of
    a persistent schedule, and per create + post + wait + delete of a fresh one (the reference's
    evaluation/allreduce.c cycle)."""
    import ctypes as C
    lib = R.lib()
    lib.rt_bench_allreduce.argtypes = [C.c_int, C.c_int64, C.c_int, C.c_int, C.POINTER(C.c_double)]
    out = {}
    for name, fresh, n in (("persistent", 0, iters), ("fresh", 1, max(iters, 256))):
        v = (C.c_double * 3)()
        if lib.rt_bench_allreduce(ranks, count, n, fresh, v) != 0:
            raise RuntimeError("native benchmark failed")
        out[name + "_us"] = v[0]
        out["correct"] = out.get("correct", True) and v[2] == 1.0
        if not fresh:
            out["first_create_us"] = v[1]
    return out


def run_sgd_loops(ranks: int, count: int, iters: int, skew_us: int = 1000) -> dict:
    """The reference's skewed SGD-loop programs (fflib2 evaluation/ssgd.c, rsgd.c, randomsgd.c) on this runtime's
    synchronous, solo and majority allreduce schedules: microseconds per post + wait, averaged over ranks, with
    rank r arriving r * skew_us late in every iteration; and how many ranks put something fresh into a round."""
    import ctypes as C
    lib = R.lib()
    lib.rt_bench_partial.argtypes = [C.c_int, C.c_int64, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_double)]
    out = {"ranks": ranks, "floats": count, "iters": iters, "skew": "rank * %d us per iteration" % skew_us}
    for mode, name in enumerate(("ssgd", "rsgd", "randomsgd")):
        v = (C.c_double * 3)()
        if lib.rt_bench_partial(ranks, count, iters, mode, skew_us, v) != 0:
            raise RuntimeError("native benchmark failed")
        out[name + "_us"], out[name + "_contributors"] = v[0], v[1]
        out["sane"] = out.get("sane", True) and v[2] == 1.0
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--ranks", type=int, default=4)
    ap.add_argument("--count", type=int, default=1024)
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--python-threads", action="store_true",
                    help="drive the ranks from Python threads (measures the binding and the interpreter as well)")
    ap.add_argument("--sgd-loops", action="store_true",
                    help="the skewed SGD loops of the reference (synchronous / solo / majority allreduce schedules)")
    ap.add_argument("--skew-us", type=int, default=1000)
    args = ap.parse_args(argv)
    if args.sgd_loops:
        print(json.dumps(run_sgd_loops(args.ranks, args.count, args.iters, args.skew_us)))
        return 0
    res = run(args.ranks, args.count, args.iters) if args.python_threads else \
        dict(ranks=args.ranks, count=args.count, dtype="int32", iters=args.iters, native=run_native(args.ranks, args.count, args.iters))
    print(json.dumps(res))
    return 0


if __name__ == "__main__":
    sys.exit(main())
