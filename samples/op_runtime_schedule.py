"""Program the host operation runtime directly: a persistent allreduce schedule with a completion
callback, re-posted with new data, and a bounded-staleness limiter.

    python samples/op_runtime_schedule.py [--ranks 4]

Ranks are threads of this process.  The primitives correspond to the reference's fflib2 API
(ff.h:106-165: ops with dependencies, schedules, ffallreduce, ffsolo_limiter).
"""
import argparse
import os
import sys
import threading

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from eagersgd_b200.parallel import oprt as R  # noqa: E402


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--ranks", type=int, default=4)
    args = ap.parse_args(argv)
    results = {}
    with R.World(args.ranks) as w:
        def body(r):
            grad = np.zeros(8, dtype=np.float32)
            total = np.zeros(8, dtype=np.float32)
            sched = r.allreduce(r.buffer(grad), r.buffer(total), tag=1)
            done = []
            cb = r.callback(lambda op: done.append(1), R.DEP_OR)
            r.hb(r.schedule_end(sched), cb)
            for step in range(3):                       # the same schedule, posted three times
                grad[:] = r.id + step
                r.schedule_post(sched)
                r.wait(cb)
            results[r.id] = (total.copy(), len(done))
            if r.id == 0:
                print(r.schedule_dot(sched).splitlines()[0], "... (%d lines of DOT)" % len(r.schedule_dot(sched).splitlines()))
        threads = [threading.Thread(target=body, args=(w.ranks[i],)) for i in range(w.n)]
        [t.start() for t in threads]
        [t.join() for t in threads]
    expect = sum(range(args.ranks)) + 2 * args.ranks
    for rid, (total, fired) in sorted(results.items()):
        assert np.all(total == expect) and fired == 3, (rid, total, fired)
    print("allreduce over %d ranks, 3 posts of one persistent schedule: sum = %g on every rank" % (args.ranks, expect))


if __name__ == "__main__":
    main()
