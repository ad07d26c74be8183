"""Program the host operation runtime directly: a persistent allreduce schedule with a completion
callback, re-posted with new data, and then a solo allreduce schedule in which the last rank is
always late and nobody waits for it.

    python samples/op_runtime_schedule.py [--ranks 4]

Ranks are threads of this process.  The primitives correspond to the reference's fflib2 API
(ff.h:106-165: ops with dependencies, schedules, ffallreduce, ffsolo_allreduce and its limiter).
"""
import argparse
import os
import sys
import threading
import time

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
        # a solo allreduce: whoever posts first starts the round everywhere (evaluation/rsgd.c:77-113)
        solo = {}
        gate = threading.Barrier(w.n)

        def solo_body(r):
            grad, avg = np.ones(8, dtype=np.float32), np.zeros(8, dtype=np.float32)
            s = r.solo_allreduce(r.buffer(grad), r.buffer(avg), tag=2, limiter=4)   # every fifth round waits for all
            waited, seen, latest = 0.0, {}, np.zeros(8, dtype=np.float32)

            def round_ended(op):                        # runs on the rank's progress thread after every round
                contributors, rnd = r.partial_read(s, latest)
                seen[rnd] = contributors
            watcher = r.callback(round_ended, R.DEP_OR)
            r.hb(r.schedule_end(s), watcher)
            r.schedule_start(s)
            for step in range(10):
                if r.id == w.n - 1:
                    time.sleep(0.01)                    # the straggler
                r.schedule_post(s)
                t0 = time.perf_counter()
                r.schedule_wait(s)
                waited += time.perf_counter() - t0
            while r.completions(watcher) < 10:
                time.sleep(0.001)
            gate.wait()
            solo[r.id] = (waited, [seen[k] for k in range(10)], r.partial_info(s))
            r.schedule_delete(s)
        threads = [threading.Thread(target=solo_body, args=(w.ranks[i],)) for i in range(w.n)]
        [t.start() for t in threads]
        [t.join() for t in threads]
    if args.ranks > 1:
        info = solo[0][2]
        assert info["rounds"] == 10 and info["sync_rounds"] == 2
        assert all(v[1] == solo[0][1] for v in solo.values())          # every rank saw the same rounds
        assert solo[0][1][4] == solo[0][1][9] == args.ranks             # the synchronous ones had everybody
        print("solo allreduce, 10 rounds, last rank 10 ms late each time: rank 0 waited %.1f ms in all "
              "(2 synchronous rounds), fresh contributors per round: %s; the late rank found %d of its "
              "rounds already begun" % (1e3 * solo[0][0], solo[0][1], solo[args.ranks - 1][2]["late"]))
    expect = sum(range(args.ranks)) + 2 * args.ranks
    for rid, (total, fired) in sorted(results.items()):
        assert np.all(total == expect) and fired == 3, (rid, total, fired)
    print("allreduce over %d ranks, 3 posts of one persistent schedule: sum = %g on every rank" % (args.ranks, expect))


if __name__ == "__main__":
    main()
