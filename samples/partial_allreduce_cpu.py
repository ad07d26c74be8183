"""The partial allreduce by itself, on CPU threads: who contributes when ranks arrive at different times.

    python samples/partial_allreduce_cpu.py [--mode solo|majority|sync] [--ranks 4] [--steps 12]

One rank per step is delayed.  In solo mode the round opens when the first rank arrives, the late rank's
gradient is picked up (stale) by the next round and the result it missed waits in its mailbox; in sync
mode everybody waits.  The evaluation programs of the reference (fflib2 evaluation/solo_allreduce*.c,
rand_allreduce*.c) print the same kind of per-step record.
"""
import argparse
import os
import sys
import threading
import time

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from eagersgd_b200.parallel.cpu_channel import CpuChannel, LocalSegments  # noqa: E402


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", default="solo")
    ap.add_argument("--ranks", type=int, default=4)
    ap.add_argument("--steps", type=int, default=12)
    ap.add_argument("--delay-ms", type=float, default=20.0)
    ap.add_argument("--accumulate", action="store_true",
                    help="fold a gradient that no round picked up into the rank's next publish instead of dropping it")
    args = ap.parse_args(argv)
    P, n = args.ranks, 16
    segs = LocalSegments(P, n, np.float32)
    totals = [np.zeros(n, dtype=np.float64) for _ in range(P)]
    dropped = [0] * P
    log = []

    def body(rank):
        ch = CpuChannel(segs.bases, rank, P, n, mode=args.mode, limiter=5, average="sum", timeout_s=30.0,
                        accumulate=args.accumulate)
        for k in range(args.steps):
            if k % P == rank:
                time.sleep(args.delay_ms / 1e3)
            out, info = ch.step(np.full(n, 1.0, dtype=np.float32))
            totals[rank] += out
            if rank == 0:
                log.append((k, int(info.role), int(info.n_contrib), int(info.is_sync)))
        out, _ = ch.flush()
        totals[rank] += out
        dropped[rank] = ch.stats()["dropped_grads"]

    t0 = time.time()
    th = [threading.Thread(target=body, args=(r,)) for r in range(P)]
    [t.start() for t in th]
    [t.join() for t in th]
    for k, role, nc, sync in log:
        print("rank 0 step %2d: role %d, %d contributions%s" % (k, role, nc, "  (synchronous round)" if sync else ""))
    print("mode %s: %d steps on %d ranks in %.0f ms" % (args.mode, args.steps, P, 1e3 * (time.time() - t0)))
    # no round result is lost: every rank has applied the same total.  A gradient that its owner replaced by a
    # newer one before any round picked it up is superseded (the reference overwrites its send buffer the same
    # way); the limiter's synchronous rounds bound how far a rank can fall behind.
    assert all(np.allclose(t, totals[0]) for t in totals), [t[0] for t in totals]
    # still sitting in a publish slot when the run ended: at most the last two gradients of every rank
    pending = P * args.steps - int(round(totals[0][0])) - sum(dropped)
    print("every rank applied the same total: %.0f of %d published gradients, %d superseded, %d still pending"
          % (totals[0][0], P * args.steps, sum(dropped), pending))
    assert 0 <= pending and (args.accumulate or pending <= 2 * P)   # a folded slot holds several gradients
    assert not (args.accumulate and sum(dropped))
    segs.close()


if __name__ == "__main__":
    main()
