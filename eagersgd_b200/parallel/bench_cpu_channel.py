"""Latency of the partial allreduce on the CPU backend under the protocol of the reference's SGD-loop programs.

    python -m eagersgd_b200.parallel.bench_cpu_channel [--ranks 2,4] [--counts 1024,262144,6553600] [--iters 12]

Every rank sleeps ``rank * 1 ms`` before each iteration (the skew of fflib2 evaluation/ssgd.c:66, rsgd.c:80,
randomsgd.c:80), then times one collective on a float vector; per iteration the mean over ranks is taken, and the mean
of those (after two warm-up iterations) is reported in microseconds — the figure the reference's programs print.
``sync`` stands where ssgd.c calls ``MPI_Allreduce``, ``solo`` where rsgd.c posts ``ffsolo_allreduce`` (limiter 1024),
``majority`` where randomsgd.c posts ``ffrand_allreduce``.  Ranks are threads of this process on the shared-memory
channel (the same code path processes take over POSIX shared memory); one JSON line per rank count and size.
"""
from __future__ import annotations

import argparse
import json
import sys
import threading
import time

import numpy as np

from .cpu_channel import CpuChannel, LocalSegments


def run(ranks: int, count: int, mode: str, iters: int = 12) -> float:
    seg = LocalSegments(ranks, count, np.float32)
    lat = [[0.0] * iters for _ in range(ranks)]
    bar = threading.Barrier(ranks)

    def body(r):
        ch = CpuChannel(seg.bases, r, ranks, count, np.float32, mode=mode, limiter=1024, average="sum", timeout_s=60.0)
        g, out = np.ones(count, np.float32), np.empty(count, np.float32)
        bar.wait()
        for it in range(iters):
            time.sleep(r * 1e-3)
            t0 = time.perf_counter()
            ch.step(g, out)
            lat[r][it] = time.perf_counter() - t0
        bar.wait()
        ch.flush(out)

    th = [threading.Thread(target=body, args=(r,)) for r in range(ranks)]
    [t.start() for t in th]
    [t.join() for t in th]
    seg.close()
    per_iter = [sum(lat[r][it] for r in range(ranks)) / ranks for it in range(2, iters)]
    return 1e6 * sum(per_iter) / len(per_iter)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--ranks", default="2,4")
    ap.add_argument("--counts", default="1024,262144,6553600")
    ap.add_argument("--iters", type=int, default=12)
    a = ap.parse_args(argv)
    for p in (int(x) for x in a.ranks.split(",")):
        for c in (int(x) for x in a.counts.split(",")):
            row = {"ranks": p, "floats": c, "bytes": 4 * c, "skew": "sleep(rank * 1 ms) per iteration"}
            for mode in ("sync", "solo", "majority"):
                row[mode + "_us"] = round(run(p, c, mode, a.iters), 1)
            print(json.dumps(row), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
