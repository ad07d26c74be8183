"""Solo and majority allreduce as schedules of the host runtime (fflib2 src/colls/ffsolo_allreduce.c,
ffrand_allreduce.c; driven like evaluation/rsgd.c and randomsgd.c: start once, then post / wait per step).

Ranks are threads.  A rank contributes ``rank + 1`` in every element, so a round's value names its contributors:
it is the sum of ``r + 1`` over the ranks that put something fresh in, and the runtime's own count of fresh
contributors has to agree with it."""
import itertools
import threading
import time

import numpy as np
import pytest

from eagersgd_b200.parallel import oprt as R


def _run(world, fn):
    errs = []

    def wrap(rank):
        try:
            fn(rank)
        except Exception:  # noqa
            import traceback
            errs.append(traceback.format_exc())
    th = [threading.Thread(target=wrap, args=(world.ranks[r],)) for r in range(world.n)]
    [t.start() for t in th]
    [t.join() for t in th]
    assert not errs, errs[0]


def _subset_sums(world):
    """value -> set of possible contributor counts, for contributions r + 1."""
    out = {}
    for k in range(world + 1):
        for sub in itertools.combinations(range(world), k):
            out.setdefault(sum(r + 1 for r in sub), set()).add(k)
    return out


def _observe(r, s, rcv, log):
    """Record (round, value, contributors) at every round end, on the progress thread, before the next round."""
    def seen(op):
        k, rnd = r.partial_read(s, rcv_copy)
        assert np.all(rcv_copy == rcv_copy[0]), rcv_copy           # one round, not a mix of two
        log.append((rnd, int(rcv_copy[0]), k))
    rcv_copy = np.zeros_like(rcv)
    cb = r.callback(seen, R.DEP_OR)
    r.hb(r.schedule_end(s), cb)

    def settled(rounds):                                            # the observer runs after the wait has returned
        t0 = time.time()
        while r.completions(cb) < rounds and time.time() - t0 < 20:
            time.sleep(0.001)
        assert r.completions(cb) == rounds
    return settled


@pytest.mark.parametrize("world", [2, 3, 4, 5])
def test_solo_rounds_agree_on_every_rank_and_lose_nothing(world):
    """Every rank sees the same value and contributor count for every round; with accumulation on and a synchronous
    last round, the rounds together contain every post exactly once."""
    steps, limiter, n = 24, 5, 17                                   # rounds 5, 11, 17, 23 are synchronous
    logs = [[] for _ in range(world)]
    infos = [None] * world
    rng = np.random.RandomState(world)
    naps = rng.uniform(0, 0.002, size=(world, steps))
    with R.World(world) as w:
        def body(r):
            snd, rcv = np.full(n, r.id + 1, dtype=np.int64), np.zeros(n, dtype=np.int64)
            s = r.solo_allreduce(r.buffer(snd), r.buffer(rcv), tag=3, limiter=limiter, options=R.PARTIAL_ACCUMULATE)
            assert s >= 0
            settled = _observe(r, s, rcv, logs[r.id])
            assert r.schedule_post(s) == R.ERROR                    # not started yet
            assert r.schedule_start(s) == R.SUCCESS
            for k in range(steps):
                time.sleep(naps[r.id, k])
                assert r.schedule_post(s) == R.SUCCESS
                snd[:] = -1000                                      # the contribution was taken inside post
                assert r.schedule_wait(s, 20.0) == R.SUCCESS
                snd[:] = r.id + 1
            settled(steps)
            w_barrier.wait()
            infos[r.id] = r.partial_info(s)
            assert r.schedule_delete(s) == R.SUCCESS
            with pytest.raises(ValueError):
                r.partial_info(s)
        w_barrier = threading.Barrier(world)
        _run(w, body)
    for log in logs:
        assert [e[0] for e in log] == list(range(steps))            # every rank ran every round, in order
    for rnd in range(steps):
        vals = {(log[rnd][1], log[rnd][2]) for log in logs}
        assert len(vals) == 1, (rnd, vals)
        value, k = vals.pop()
        assert 1 <= k <= world and value >= k                       # somebody activated it; accumulated posts may add up
        if rnd % (limiter + 1) == limiter:
            assert k == world                                       # a synchronous round has everybody
    assert sum(e[1] for e in logs[0]) == steps * sum(range(1, world + 1))
    for i in infos:
        assert i["posts"] == steps and i["rounds"] == steps and i["sync_rounds"] == 4 and i["pending"] == 0
        assert i["overwritten"] == 0
    assert sum(i["activated"] for i in infos) >= steps - 4          # each eager round had at least one activator


def test_solo_does_not_wait_for_a_slow_rank_and_the_limiter_does():
    world, steps, nap = 4, 12, 0.03
    waits = [0.0] * world
    infos = [None] * world
    logs = [[] for _ in range(world)]
    with R.World(world) as w:
        done = threading.Barrier(world)

        def body(r):
            snd, rcv = np.full(8, float(1 << r.id), dtype=np.float32), np.zeros(8, dtype=np.float32)   # a bit per rank
            s = r.solo_allreduce(r.buffer(snd), r.buffer(rcv), tag=1, limiter=-1)
            settled = _observe(r, s, rcv, logs[r.id])
            r.schedule_start(s)
            for k in range(steps):
                if r.id == 3:
                    time.sleep(nap)
                r.schedule_post(s)
                t0 = time.perf_counter()
                assert r.schedule_wait(s, 20.0) == R.SUCCESS
                waits[r.id] += time.perf_counter() - t0
            settled(steps)
            done.wait()
            infos[r.id] = r.partial_info(s)
            r.schedule_delete(s)
        t0 = time.perf_counter()
        _run(w, body)
    assert max(waits[:3]) < 0.5 * steps * nap, waits               # the on-time ranks never sat out a nap
    for rnd in range(steps):
        assert len({(log[rnd][1], log[rnd][2]) for log in logs}) == 1
        assert bin(logs[0][rnd][1]).count("1") == logs[0][rnd][2] >= 1, logs[0][rnd]   # the value names its contributors
    assert infos[3]["late"] >= steps - 2 and infos[3]["activated"] <= 2   # the slow rank found its rounds begun
    assert sum(1 for e in logs[0] if e[1] & 7) == steps             # every round had one of the on-time ranks
    for q in range(world):                                          # a post is taken by a round, replaced, or left over
        taken = sum(1 for e in logs[0] if e[1] & (1 << q))
        assert taken + infos[q]["overwritten"] + infos[q]["pending"] == steps, (q, taken, infos[q])
    assert sum(1 for e in logs[0] if e[1] & 8) <= steps // 2        # the slow rank is in few rounds, if any
    # the same loop with a limiter of 0 is a synchronous allreduce: everybody waits for the slow rank
    waits2 = [0.0] * world
    with R.World(world) as w:
        def body2(r):
            x, y = np.full(8, float(r.id + 1), dtype=np.float32), np.zeros(8, dtype=np.float32)
            s = r.solo_allreduce(r.buffer(x), r.buffer(y), tag=1, limiter=0)
            r.schedule_start(s)
            for k in range(4):
                if r.id == 3:
                    time.sleep(nap)
                r.schedule_post(s)
                t0 = time.perf_counter()
                assert r.schedule_wait(s, 20.0) == R.SUCCESS
                waits2[r.id] += time.perf_counter() - t0
                assert np.all(y == 10.0)                            # 1 + 2 + 3 + 4: nobody is missing
            r.schedule_delete(s)
        _run(w, body2)
    assert min(waits2[:3]) > 0.5 * 4 * nap, waits2


def test_majority_waits_for_the_drawn_rank_only():
    world, steps, seed = 4, 16, 77
    logs = [[] for _ in range(world)]
    infos = [None] * world
    draws = [None] * world
    with R.World(world) as w:
        done = threading.Barrier(world)

        def body(r):
            snd, rcv = np.full(4, r.id + 1, dtype=np.int32), np.zeros(4, dtype=np.int32)
            s = r.rand_allreduce(r.buffer(snd), r.buffer(rcv), tag=2, seed=seed, limiter=7)
            draws[r.id] = [r.partial_activator(s, k) for k in range(steps)]
            settled = _observe(r, s, rcv, logs[r.id])
            r.schedule_start(s)
            for k in range(steps):
                time.sleep(0.001 * r.id)
                r.schedule_post(s)
                assert r.schedule_wait(s, 20.0) == R.SUCCESS
            settled(steps)
            done.wait()
            infos[r.id] = r.partial_info(s)
            r.schedule_delete(s)
        _run(w, body)
    assert draws[0] == draws[1] == draws[2] == draws[3]             # one draw, known to everybody
    assert draws[0][7] == -1 and draws[0][15] == -1 and len(set(draws[0]) - {-1}) > 1
    for rank, i in enumerate(infos):
        assert i["activated"] <= sum(1 for d in draws[0] if d == rank)
        assert i["rounds"] == steps and i["sync_rounds"] == 2
    for rnd in range(steps):
        assert len({(log[rnd][1], log[rnd][2]) for log in logs}) == 1
        if draws[0][rnd] >= 0:                                      # the drawn rank's own contribution is in its round
            value, k = logs[0][rnd][1], logs[0][rnd][2]
            assert any(draws[0][rnd] in sub and sum(q + 1 for q in sub) == value
                       for sub in itertools.combinations(range(world), k)), (rnd, value, k)


def test_neutral_element_stale_option_and_other_operators():
    """A rank with nothing new contributes the operator's neutral element (maximum: the lowest value), or with
    PARTIAL_STALE its previous contribution once more."""
    out = {}
    with R.World(2) as w:
        gate = threading.Barrier(2)

        def body(r):
            snd = np.full(3, 10.0 * (r.id + 1))
            scheds = {"max": r.solo_allreduce(r.buffer(snd), r.buffer(np.zeros(3)), tag=4, op=R.MAX),
                      "stale": r.solo_allreduce(r.buffer(snd), r.buffer(np.zeros(3)), tag=5, options=R.PARTIAL_STALE)}
            res = np.zeros(3)

            def alone(key, rnd):                                    # rank 0 activates a round; rank 1's user is elsewhere
                if r.id == 0:
                    r.schedule_post(scheds[key])
                    assert r.schedule_wait(scheds[key], 20.0) == R.SUCCESS
                    k, got = r.partial_read(scheds[key], res)
                    assert got == rnd
                    out[key, rnd] = (res[0], k)

            def catch_up(key, n):                                   # rank 1 posts rounds that are over already
                if r.id == 1:
                    for _ in range(n):
                        r.schedule_post(scheds[key])
                        assert r.schedule_wait(scheds[key], 1.0) == R.SUCCESS

            for q in scheds.values():
                r.schedule_start(q)
            gate.wait()
            for key in scheds:
                alone(key, 0)                                       # rank 1 has posted nothing yet
            gate.wait()
            for key in scheds:
                catch_up(key, 1)                                    # its contribution of 20 now waits for a round
            gate.wait()
            for key in scheds:
                alone(key, 1)                                       # takes the 20
                alone(key, 2)                                       # nothing new from rank 1
            gate.wait()
            for key in scheds:
                catch_up(key, 2)
            gate.wait()
            for key, q in scheds.items():
                i = r.partial_info(q)
                assert i["rounds"] == 3 and i["posts"] == 3
                if r.id == 1:
                    assert i["late"] == 3 and i["activated"] == 0 and i["overwritten"] == 1 and i["pending"] == 1
                else:
                    assert i["late"] == 0 and i["activated"] == 3
                r.schedule_delete(q)
        _run(w, body)
    assert out["max", 0] == (10.0, 1) and out["stale", 0] == (10.0, 1)
    assert out["max", 1] == (20.0, 2) and out["stale", 1] == (30.0, 2)
    assert out["max", 2] == (10.0, 1)                                # the lowest value stood in for rank 1, not 0 or 20
    assert out["stale", 2] == (30.0, 1)                              # its 20 counted again, though only one was fresh


def test_create_delete_cycles_reuse_the_tag_and_a_missing_rank_times_out():
    with R.World(3) as w:
        def body(r):
            for cycle in range(40):
                x, y, res = np.full(2, r.id + 1, dtype=np.int32), np.zeros(2, dtype=np.int32), np.zeros(2, dtype=np.int32)
                bx, by = r.buffer(x), r.buffer(y)
                s = r.solo_allreduce(bx, by, tag=9, limiter=1)
                r.schedule_start(s)
                for k in range(4):
                    r.schedule_post(s)
                    assert r.schedule_wait(s, 20.0) == R.SUCCESS
                    if k % 2 == 1:                                  # a synchronous round; a peer may have begun the next
                        contributors, rnd = r.partial_read(s, res)  # one already, so ask which round the buffer holds
                        if rnd == k:
                            assert np.all(res == 6) and contributors == 3
                assert np.all(y == 6)                               # nothing follows the last round
                assert r.schedule_delete(s) == R.SUCCESS
                m = r.rand_allreduce(bx, by, tag=9, seed=cycle, limiter=3)    # the same tag again, another collective
                r.schedule_start(m)
                for k in range(4):
                    r.schedule_post(m)
                    assert r.schedule_wait(m, 20.0) == R.SUCCESS
                assert np.all(y == 6) and r.partial_info(m)["rounds"] == 4
                assert r.schedule_delete(m) == R.SUCCESS
                r.buffer_delete(bx)
                r.buffer_delete(by)
        _run(w, body)
    with R.World(2) as w:
        def body(r):
            x, y = np.ones(2, dtype=np.int32), np.zeros(2, dtype=np.int32)
            s = r.solo_allreduce(r.buffer(x), r.buffer(y), tag=1, limiter=0)
            r.schedule_start(s)
            if r.id == 0:                                           # rank 1 never posts the synchronous round
                r.schedule_post(s)
                t0 = time.perf_counter()
                assert r.schedule_wait(s, 0.3) == R.TIMEOUT
                assert time.perf_counter() - t0 < 5.0
                assert r.schedule_test(s) == R.SUCCESS              # still not complete, and nothing hangs
        _run(w, body)


def test_print_shows_the_parts():
    with R.World(2) as w:
        def body(r):
            x, y = np.ones(2, dtype=np.float32), np.zeros(2, dtype=np.float32)
            s = r.solo_allreduce(r.buffer(x), r.buffer(y), tag=1)
            dot = r.schedule_dot(s)
            assert dot.count("digraph") == 3 and dot.count("callback") >= 4 and "send" in dot and "recv" in dot
            r.schedule_delete(s)
        _run(w, body)


def test_sgd_loop_benchmark_shows_the_three_behaviours():
    """The reference's ssgd / rsgd / randomsgd loops on this runtime: with rank r arriving r ms late, the synchronous
    allreduce costs the ranks about the mean lateness, the solo allreduce next to nothing, the majority one lies between."""
    from eagersgd_b200.parallel.bench_oprt import run_sgd_loops
    r = run_sgd_loops(ranks=4, count=512, iters=42, skew_us=1000)
    assert r["sane"]
    assert r["ssgd_contributors"] == 4.0 and r["rsgd_contributors"] >= 1.0
    assert r["rsgd_us"] < 0.5 * r["ssgd_us"], r
    assert r["rsgd_us"] < r["randomsgd_us"] < 1.25 * r["ssgd_us"], r


def test_one_random_slow_rank_with_a_limiter_of_twenty():
    """evaluation/solo_allreduce_single.c / solo_allreduce_multiple.c: every rank increments its vector before each
    post, one rank drawn from a shared seed sleeps before its posts, limiter 20; nobody but that rank waits, and
    what arrives is always a whole round."""
    world, iters, n = 4, 25, 33
    slow = int(np.random.RandomState(434656342 % (2 ** 31)).randint(world))
    waits = [0.0] * world
    infos = [None] * world
    with R.World(world) as w:
        done = threading.Barrier(world)

        def body(r):
            to_reduce, reduced, res = np.zeros(n, dtype=np.int32), np.zeros(n, dtype=np.int32), np.zeros(n, dtype=np.int32)
            s = r.solo_allreduce(r.buffer(to_reduce), r.buffer(reduced), tag=0, limiter=20)
            if r.id == 0:
                assert r.schedule_dot(s).count("digraph") == 3             # the program prints the schedule first
            r.schedule_start(s)
            for it in range(iters):
                to_reduce += 1
                if r.id == slow:
                    time.sleep(0.01)
                r.schedule_post(s)
                t0 = time.perf_counter()
                assert r.schedule_wait(s, 20.0) == R.SUCCESS
                waits[r.id] += time.perf_counter() - t0
                k, rnd = r.partial_read(s, res)
                assert np.all(res == res[0]) and 0 <= k <= world and rnd >= it
            done.wait()
            infos[r.id] = r.partial_info(s)
            r.schedule_delete(s)
        _run(w, body)
    for q in range(world):
        assert infos[q]["rounds"] == iters and infos[q]["sync_rounds"] == 1        # round 20
    others = [waits[q] for q in range(world) if q != slow]
    assert infos[slow]["late"] >= iters - 6                         # the slow rank found nearly all of its rounds begun
    assert max(others) < 0.25 + 0.01 * 22                           # the others waited for it in the synchronous round only


@pytest.mark.parametrize("kind", ["solo", "majority"])
def test_several_collectives_side_by_side_on_balanced_ranks(kind):
    """evaluation/rsgd_synch_send.c, rsgd_synch_recv.c and their ssgd twins: N persistent schedules with tags 0..N-1,
    posted and waited for one after the other in every iteration; with nobody late every round has everybody."""
    world, N, iters, n = 3, 3, 10, 64
    with R.World(world) as w:
        def body(r):
            snd = [np.zeros(n, dtype=np.float32) for _ in range(N)]
            rcv = [np.zeros(n, dtype=np.float32) for _ in range(N)]
            make = (lambda i: r.solo_allreduce(r.buffer(snd[i]), r.buffer(rcv[i]), tag=i, limiter=0)) if kind == "solo" else \
                   (lambda i: r.rand_allreduce(r.buffer(snd[i]), r.buffer(rcv[i]), tag=i, seed=6545343, limiter=0))
            scheds = [make(i) for i in range(N)]
            for s in scheds:
                r.schedule_start(s)
            for it in range(iters):
                for i, s in enumerate(scheds):
                    snd[i][:] = 1.0 + i
                    r.schedule_post(s)
                    assert r.schedule_wait(s, 20.0) == R.SUCCESS
                    assert np.all(rcv[i] == world * (1.0 + i)), (it, i, rcv[i][:3])   # limiter 0: every round has all ranks
                    snd[i][:] = 0.0
            for s in scheds:
                assert r.partial_info(s)["rounds"] == iters
                r.schedule_delete(s)
        _run(w, body)


def test_a_rank_that_posts_ahead_cannot_pull_others_across_a_synchronous_round():
    """Rank 0 posts four rounds without waiting in between (limiter 1: rounds 1 and 3 are synchronous).  Its token for
    round 2 reaches rank 1 before rank 1 has posted round 1; rank 1 must not begin rounds 1 and 2 on the token's word —
    round 1 has to contain rank 1's own contribution."""
    log = [[], []]
    with R.World(2) as w:
        gate = threading.Barrier(2)

        def body(r):
            snd, rcv = np.full(4, 1 << r.id, dtype=np.int32), np.zeros(4, dtype=np.int32)
            s = r.solo_allreduce(r.buffer(snd), r.buffer(rcv), tag=6, limiter=1)
            settled = _observe(r, s, rcv, log[r.id])
            r.schedule_start(s)
            gate.wait()
            if r.id == 0:
                for _ in range(4):
                    assert r.schedule_post(s) == R.SUCCESS
                time.sleep(0.05)                                # rank 1 has seen whatever tokens there are
                gate.wait()
                for _ in range(4):
                    assert r.schedule_wait(s, 20.0) == R.SUCCESS
            else:
                gate.wait()
                assert r.partial_info(s)["rounds"] == 1         # round 0 ran on the token; round 1 waits for the post
                for _ in range(4):
                    r.schedule_post(s)
                    assert r.schedule_wait(s, 20.0) == R.SUCCESS
            settled(4)
            gate.wait()
            r.schedule_delete(s)
        _run(w, body)
    assert [e[:2] for e in log[0]] == [e[:2] for e in log[1]]
    values = [e[1] for e in log[0]]
    assert values[1] & 2 and values[3] & 2, log[0]               # rank 1 is in both synchronous rounds
    # (rank 0's four posts came faster than the rounds could take them: some of its contributions replaced each other)


@pytest.mark.parametrize("kind,world", [("solo", 2), ("solo", 3), ("solo", 5), ("majority", 4)])
def test_fenced_rounds_equal_a_full_allreduce(kind, world):
    """evaluation/solo_allreduce_correctness.c and rand_allreduce_correctness.c: every rank increments its vector, then
    barrier, post, wait, barrier; with the rounds fenced like this everybody's data is in every round, so the result
    must equal a plain allreduce of the vectors.  PARTIAL_LIVE gives the reference's semantics (a round reads the send
    buffer when it begins); without it the same holds once the rounds are counted together with what a late post left
    for the next one, which is what the last, synchronous round shows."""
    iters, n = 21, 19
    with R.World(world) as w:
        fence = threading.Barrier(world)

        def body(r):
            to_reduce, reduced, res = np.zeros(n, dtype=np.int32), np.zeros(n, dtype=np.int32), np.zeros(n, dtype=np.int32)
            make = r.solo_allreduce if kind == "solo" else (lambda *a, **k: r.rand_allreduce(*a, seed=34495645 % (2 ** 31), **k))
            s = make(r.buffer(to_reduce), r.buffer(reduced), tag=0, limiter=20, options=R.PARTIAL_LIVE)
            r.schedule_start(s)
            for it in range(iters):
                to_reduce += 1
                fence.wait()
                r.schedule_post(s)
                assert r.schedule_wait(s, 20.0) == R.SUCCESS
                fence.wait()
                k, rnd = r.partial_read(s, res)
                assert rnd == it and np.all(res == world * (it + 1)), (r.id, it, rnd, res[:3])
                assert np.array_equal(reduced, res)
                fence.wait()
            info = r.partial_info(s)
            assert info["rounds"] == iters and info["sync_rounds"] == 1
            r.schedule_delete(s)
        _run(w, body)


@pytest.mark.parametrize("kind", ["solo", "majority"])
def test_three_imbalance_regimes_keep_every_contribution(kind):
    """evaluation/ssgd_synch_send.c, rsgd_synch_send.c and their _recv twins: a balanced phase, a phase in which two
    ranks drawn anew in every iteration sleep, and a phase in which ranks 0 and 1 always sleep.  Those programs print
    the reduced arrays for the reader to judge; here the invariants are asserted: every rank runs every round and sees
    the same rounds; with accumulation on, the rounds up to each synchronous one hold every post made until then exactly
    once; and in the constant phase the ranks that are never late do not wait for the two that always are (solo)."""
    world, per_phase, limiter, nap = 4, 12, 5, 0.004               # 36 rounds; 5, 11, 17, ... are synchronous
    steps = 3 * per_phase
    rng = np.random.RandomState(6545343 % (2 ** 31))
    sleepers = [set()] * per_phase + [set(rng.choice(world, 2, replace=False).tolist()) for _ in range(per_phase)] + \
               [{0, 1}] * per_phase
    logs = [[] for _ in range(world)]
    waits = np.zeros((world, 3))
    with R.World(world) as w:
        gate = threading.Barrier(world)

        def body(r):
            snd, rcv = np.full(8, 1 << (8 * r.id), dtype=np.int64), np.zeros(8, dtype=np.int64)   # a byte per rank
            opts = dict(tag=0, limiter=limiter, options=R.PARTIAL_ACCUMULATE)
            s = r.solo_allreduce(r.buffer(snd), r.buffer(rcv), **opts) if kind == "solo" else \
                r.rand_allreduce(r.buffer(snd), r.buffer(rcv), seed=6545343 % (2 ** 31), **opts)
            settled = _observe(r, s, rcv, logs[r.id])
            r.schedule_start(s)
            gate.wait()
            for it in range(steps):
                if r.id in sleepers[it]:
                    time.sleep(nap)
                r.schedule_post(s)
                t0 = time.perf_counter()
                assert r.schedule_wait(s, 20.0) == R.SUCCESS
                waits[r.id, it // per_phase] += time.perf_counter() - t0
            settled(steps)
            gate.wait()
            info = r.partial_info(s)
            assert info["rounds"] == steps and info["overwritten"] == 0 and info["pending"] == 0
            r.schedule_delete(s)
        _run(w, body)
    for q in range(1, world):
        assert logs[q] == logs[0]                                   # every rank saw the same rounds
    total = 0
    for rnd, value, k in logs[0]:
        total += value
        if rnd % (limiter + 1) == limiter:                          # a synchronous round: everybody has posted rnd + 1 times
            assert k == world
            assert [(total >> (8 * q)) & 0xff for q in range(world)] == [rnd + 1] * world, (rnd, hex(total))
    if kind == "solo":
        # ranks 2 and 3 are never late in the constant phase; they wait only in its two synchronous rounds
        assert waits[2:, 2].max() < 2 * (limiter + 1) * nap + 0.25 * per_phase * nap + 0.05, waits


@pytest.mark.parametrize("kind", ["solo", "majority"])
def test_a_world_of_one_rank(kind):
    with R.World(1) as w:
        r = w.ranks[0]
        x, y, res = np.arange(5, dtype=np.float64), np.zeros(5), np.zeros(5)
        s = r.solo_allreduce(r.buffer(x), r.buffer(y), 0, limiter=2) if kind == "solo" else \
            r.rand_allreduce(r.buffer(x), r.buffer(y), 0, seed=1, limiter=2)
        r.schedule_start(s)
        for it in range(7):
            x[:] = np.arange(5) + it
            assert r.schedule_post(s) == R.SUCCESS and r.schedule_wait(s, 5.0) == R.SUCCESS
            k, rnd = r.partial_read(s, res)
            assert (k, rnd) == (1, it) and np.array_equal(res, np.arange(5) + it)
        i = r.partial_info(s)
        assert (i["rounds"], i["sync_rounds"], i["late"], i["pending"]) == (7, 2, 0, 0)
        assert r.schedule_delete(s) == R.SUCCESS
