"""Step time of synchronous, majority and solo averaging when every rank's compute time varies from step to step.

    python samples/imbalance_modes_cpu.py [--ranks 4] [--steps 60] [--buckets 6]

Ranks are threads on the CPU backend; each step a rank "computes" for a random 4 to 12 ms and then averages its
gradient buckets.  Synchronous averaging makes every step as long as the slowest rank's; solo lets each rank go on
with whoever has arrived (bounded by the limiter); majority waits for one designated rank per round.  This is the
natural-imbalance setting of the reference's video workload (variable-length sequences) reduced to its timing.
"""
import argparse
import os
import random
import sys
import threading
import time

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from eagersgd_b200.parallel.cpu_channel import CpuChannel, LocalSegments  # noqa: E402


def run(ranks, mode, steps, buckets, count=4096, limiter=32, lo=0.004, hi=0.012):
    segs = [LocalSegments(ranks, count, np.float32) for _ in range(buckets)]
    bar = threading.Barrier(ranks)
    total, comm = [0.0] * ranks, [0.0] * ranks

    def body(r):
        chans = [CpuChannel(s.bases, r, ranks, count, np.float32, mode=mode, limiter=limiter, timeout_s=30.0)
                 for s in segs]
        rng = random.Random(100 + r)
        g, out = np.ones(count, np.float32), np.empty(count, np.float32)
        bar.wait()
        t0 = time.perf_counter()
        for _ in range(steps):
            time.sleep(lo + (hi - lo) * rng.random())
            tw = time.perf_counter()
            for ch in chans:
                ch.step(g, out)
            comm[r] += time.perf_counter() - tw
        total[r] = time.perf_counter() - t0
        bar.wait()
        for ch in chans:
            ch.flush(out)

    th = [threading.Thread(target=body, args=(r,)) for r in range(ranks)]
    [t.start() for t in th]
    [t.join() for t in th]
    return 1e3 * max(total) / steps, 1e3 * sum(comm) / ranks / steps


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ranks", type=int, default=4)
    ap.add_argument("--steps", type=int, default=60)
    ap.add_argument("--buckets", type=int, default=6)
    a = ap.parse_args()
    res = {}
    for mode in ("sync", "majority", "solo"):
        res[mode] = run(a.ranks, mode, a.steps, a.buckets)
        print("%-8s %6.2f ms per step (of which averaging + waiting %5.2f ms)" % ((mode,) + res[mode]))
    assert res["solo"][1] < res["sync"][1], "solo should spend less time in the collective than sync"
    print("mean compute time per step is 8 ms; the rest is what the collective costs each mode")


if __name__ == "__main__":
    main()
