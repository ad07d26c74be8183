"""Partial-allreduce protocol on the CPU backend, ranks as threads of one process.

Mirrors the reference's evaluation programs with assertable invariants
(fflib2 evaluation/solo_allreduce_correctness.c, rand_allreduce_correctness.c,
allreduce.c, limiter.c, solo_allreduce_multiple.c): closed-form sums for the
synchronous mode at 1..8 ranks including non-powers of two, and, for the eager
modes under random delays, (a) untorn results, (b) identical accumulated
updates on every rank, (c) the limiter's sync pattern.
"""
import random
import threading
import time

import numpy as np
import pytest

from eagersgd_b200.parallel import _native as N
from eagersgd_b200.parallel.cpu_channel import CpuChannel, LocalSegments


def _run(world, mode, limiter, steps, count=512, dtype=np.float64, delay=0.002, seed=0, average="sum",
         include_stale=True, slow_rank=None):
    segs = LocalSegments(world, count, dtype)
    applied = [np.zeros(count, dtype=np.float64) for _ in range(world)]
    infos = [[] for _ in range(world)]
    errors = []

    def worker(r):
        try:
            ch = CpuChannel(segs.bases, r, world, count, dtype, mode=mode, limiter=limiter, seed=99,
                            average=average, include_stale=include_stale, timeout_s=30)
            rng = random.Random(seed * 131 + r)
            for k in range(1, steps + 1):
                if delay and (rng.random() < 0.3 or r == slow_rank):
                    time.sleep(rng.random() * delay)
                g = np.full(count, (r + 1) * 1000 + k, dtype=dtype)
                out, info = ch.step(g)
                assert np.all(out == out[0]), "torn result"
                applied[r] += out
                infos[r].append((info.role, info.round, info.n_contrib, info.n_fresh, info.is_sync))
        except Exception as e:  # noqa
            errors.append((r, repr(e)))

    th = [threading.Thread(target=worker, args=(r,)) for r in range(world)]
    [t.start() for t in th]
    [t.join() for t in th]
    assert not errors, errors
    stats = []
    for r in range(world):
        ch = CpuChannel(segs.bases, r, world, count, dtype, mode=mode, limiter=limiter, seed=99, average=average,
                        timeout_s=10)
        out, info = ch.flush()
        applied[r] += out
        stats.append(ch.stats())
    return applied, infos, stats


@pytest.mark.parametrize("world", [1, 2, 3, 4, 5, 8])
def test_sync_closed_form(world):
    steps = 25
    applied, infos, _ = _run(world, "sync", -1, steps, dtype=np.int64, delay=0.001)
    total = sum((r + 1) * 1000 + k for r in range(world) for k in range(1, steps + 1))
    for r in range(world):
        assert applied[r][0] == total
        assert all(i[0] == N.ROLE_PARTICIPANT and i[2] == world for i in infos[r])


@pytest.mark.parametrize("dtype", [np.float32, np.float64, np.int32, np.int64])
def test_sync_datatypes(dtype):
    applied, _, _ = _run(3, "sync", -1, 5, dtype=dtype, delay=0)
    total = sum((r + 1) * 1000 + k for r in range(3) for k in range(1, 6))
    assert applied[0][0] == total


@pytest.mark.parametrize("mode", ["solo", "majority"])
@pytest.mark.parametrize("world", [2, 3, 4, 8])
def test_eager_replicas_agree(mode, world):
    """Every rank ends with the same sum of round results: nothing a round produced is lost."""
    applied, infos, stats = _run(world, mode, -1, 60)
    for r in range(1, world):
        assert np.array_equal(applied[r], applied[0])
    published = sum((r + 1) * 1000 + k for r in range(world) for k in range(1, 61))
    assert 0 < applied[0][0] <= published  # a superseded gradient may be dropped, never duplicated
    assert all(s["status"] == 0 for s in stats)


def test_limiter_pattern_and_exactness():
    """limiter=3: steps 4, 8, 12 ... are synchronous with every rank contributing."""
    world, steps = 4, 24
    applied, infos, stats = _run(world, "solo", 3, steps)
    for r in range(world):
        for k, info in enumerate(infos[r], start=1):
            if k % 4 == 0:
                assert info[4] == 1 and info[0] == N.ROLE_PARTICIPANT and info[2] == world and info[1] == k
            else:
                assert info[4] == 0
        assert stats[r]["sync_rounds"] == steps // 4
    for r in range(1, world):
        assert np.array_equal(applied[r], applied[0])


def test_limiter_zero_is_synchronous():
    applied, _, _ = _run(3, "solo", 0, 10, dtype=np.int64)
    assert applied[0][0] == sum((r + 1) * 1000 + k for r in range(3) for k in range(1, 11))


def test_solo_does_not_wait_for_a_slow_rank():
    """A constantly slow rank must not hold the others back (solo_allreduce_multiple.c)."""
    world, steps, count = 3, 12, 64
    segs = LocalSegments(world, count, np.float32)
    t_done = [0.0] * world

    def worker(r):
        ch = CpuChannel(segs.bases, r, world, count, np.float32, mode="solo", limiter=-1, timeout_s=30)
        for k in range(steps):
            if r == 2:
                time.sleep(0.03)
            ch.step(np.ones(count, dtype=np.float32))
        t_done[r] = time.time()

    t0 = time.time()
    th = [threading.Thread(target=worker, args=(r,)) for r in range(world)]
    [t.start() for t in th]
    [t.join() for t in th]
    assert min(t_done[0], t_done[1]) - t0 < 0.5 * (t_done[2] - t0)


def test_majority_initiator_stream_is_shared():
    lib = N.host()
    seq = [lib.esgd_majority_initiator(6545343, k, 8) for k in range(1, 200)]
    assert set(seq) == set(range(8))
    assert seq == [lib.esgd_majority_initiator(6545343, k, 8) for k in range(1, 200)]


def test_averaging_modes():
    for average, expect in (("world", lambda s, n, w: s / w), ("contributors", lambda s, n, w: s / n)):
        world, count = 4, 16
        segs = LocalSegments(world, count, np.float32)
        outs = [None] * world

        def worker(r):
            ch = CpuChannel(segs.bases, r, world, count, np.float32, mode="sync", limiter=-1, average=average)
            outs[r], _ = ch.step(np.full(count, r + 1.0, dtype=np.float32))

        th = [threading.Thread(target=worker, args=(r,)) for r in range(world)]
        [t.start() for t in th]
        [t.join() for t in th]
        for r in range(world):
            assert np.allclose(outs[r], 10.0 / 4)


def test_dead_rank_times_out_with_status():
    """Failure detection on the host: a rank that never joins a synchronous round
    makes the others' bounded wait run out with an error status."""
    world, count = 2, 16
    segs = LocalSegments(world, count, np.float32)
    ch = CpuChannel(segs.bases, 0, world, count, np.float32, mode="sync", limiter=-1, timeout_s=0.3)
    with pytest.raises(N.ChannelError) as e:
        ch.step(np.ones(count, dtype=np.float32))
    assert e.value.status & 3       # the round never opened, or it opened and a rank never arrived


def test_trace_ring_and_watchdog():
    """The trace ring records role / round / masks per step; the watchdog turns a status word into an error."""
    from eagersgd_b200.parallel.watchdog import Watchdog
    world, count = 2, 16
    segs = LocalSegments(world, count, np.float32)
    chans = [CpuChannel(segs.bases, r, world, count, np.float32, mode="sync", limiter=-1, timeout_s=5) for r in range(world)]
    th = [threading.Thread(target=lambda c=c: [c.step(np.ones(count, dtype=np.float32)) for _ in range(5)]) for c in chans]
    [t.start() for t in th]
    [t.join() for t in th]
    tr = chans[0].trace()
    assert [e["step"] for e in tr] == [1, 2, 3, 4, 5]
    assert all(e["role"] == "participant" and e["fresh_mask"] == 3 and e["is_sync"] == 1 for e in tr)

    class FakeOpt:
        def check(self_inner):
            raise N.ChannelError(2, "fake")
    seen = []
    wd = Watchdog(FakeOpt(), period_s=0.05, on_failure=seen.append).start()
    time.sleep(0.3)
    wd.stop()
    assert seen and seen[0].status == 2
    with pytest.raises(N.ChannelError):
        wd.raise_if_failed()


@pytest.mark.parametrize("mode", ["solo", "majority"])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_accumulate_loses_no_gradient(mode, world):
    """With ``accumulate`` a gradient that no round picked up is folded into the rank's next publish of
    the same slot: after two closing synchronous rounds every published gradient has been applied exactly
    once on every rank (the reference drops such gradients: opt_esgd_solo_imagenet_imbalance.py:301-314)."""
    count, steps = 64, 50
    segs = LocalSegments(world, count, np.int64)
    applied = [np.zeros(count, dtype=np.int64) for _ in range(world)]
    stats = [None] * world
    errors = []
    phase = threading.Barrier(world)      # every rank changes the channel's mode at the same point

    def worker(r):
        try:
            kw = dict(seed=99, average="sum", timeout_s=30, accumulate=True)
            ch = CpuChannel(segs.bases, r, world, count, np.int64, mode=mode, limiter=-1, **kw)
            rng = random.Random(7 * world + r)
            for k in range(1, steps + 1):
                if rng.random() < 0.4 or r == 0:
                    time.sleep(rng.random() * 0.003)
                out, _ = ch.step(np.full(count, (r + 1) * 1000 + k, dtype=np.int64))
                assert np.all(out == out[0])
                applied[r] += out
            phase.wait()
            closing = CpuChannel(segs.bases, r, world, count, np.int64, mode="sync", limiter=-1, **kw)
            for _ in range(2):   # both slot parities are flushed
                out, _ = closing.step(np.zeros(count, dtype=np.int64))
                applied[r] += out
            stats[r] = closing.stats()
        except Exception as e:  # noqa
            errors.append((r, repr(e)))

    th = [threading.Thread(target=worker, args=(r,)) for r in range(world)]
    [t.start() for t in th]
    [t.join() for t in th]
    assert not errors, errors
    published = sum((r + 1) * 1000 + k for r in range(world) for k in range(1, steps + 1))
    for r in range(world):
        assert applied[r][0] == published, (r, applied[r][0], published)
        assert stats[r]["status"] == 0 and stats[r]["dropped_grads"] == 0
    assert sum(s["folded_grads"] for s in stats) > 0      # the case did occur


def test_adaptive_grace_window_tracks_arrival_spread():
    """Ranks arriving within a few hundred microseconds of each other end up in the same round once the
    activators have learnt the spread; the window never exceeds ``grace_us``."""
    world, count, steps = 3, 16, 40
    segs = LocalSegments(world, count, np.float32)
    fresh = [[] for _ in range(world)]
    barrier = threading.Barrier(world)

    def worker(r):
        ch = CpuChannel(segs.bases, r, world, count, np.float32, mode="solo", limiter=-1, timeout_s=30,
                        grace_us=20000.0, adaptive_grace=True)
        for k in range(steps):
            barrier.wait()
            time.sleep(0.0003 * r)
            _, info = ch.step(np.ones(count, dtype=np.float32))
            fresh[r].append(info.n_fresh if info.role == N.ROLE_PARTICIPANT else 0)

    th = [threading.Thread(target=worker, args=(r,)) for r in range(world)]
    [t.start() for t in th]
    [t.join() for t in th]
    assert sum(1 for f in fresh[0][20:] if f == world) >= 10


def test_cpu_channel_benchmark_runs_the_skewed_loop():
    """The SGD-loop protocol of the reference's timing programs on the CPU backend: a late rank costs the solo
    collective nothing, the synchronous one its lateness."""
    from eagersgd_b200.parallel.bench_cpu_channel import run
    solo = run(2, 1024, "solo", iters=6)
    sync = run(2, 1024, "sync", iters=6)
    assert 0 < solo < sync and sync > 300.0      # rank 1 sleeps 1 ms: the mean wait of two ranks is about 500 us


@pytest.mark.parametrize("mode", ["sync", "solo"])
def test_large_vectors_on_several_threads_per_rank(mode):
    """Vectors large enough for the rank's helper threads (from 256 K elements per thread), with a length that is
    no multiple of the reduction block: position-dependent values come out summed element by element, replicas
    agree in the eager mode, nothing is torn at the thread boundaries."""
    world, count, steps = 2, (1 << 20) + 12345, 4
    segs = LocalSegments(world, count, np.float32)
    base = (np.arange(count) % 97).astype(np.float32)
    applied = [np.zeros(count, dtype=np.float64) for _ in range(world)]
    errors = []

    def worker(r):
        try:
            ch = CpuChannel(segs.bases, r, world, count, np.float32, mode=mode, limiter=2, average="sum", timeout_s=60)
            for k in range(1, steps + 1):
                if mode == "solo" and r == 1:
                    time.sleep(0.003)
                out, info = ch.step(base * (r + 1) + k)
                applied[r] += out
            out, _ = ch.flush()
            applied[r] += out
        except Exception as e:  # noqa
            errors.append((r, repr(e)))

    th = [threading.Thread(target=worker, args=(r,)) for r in range(world)]
    [t.start() for t in th]
    [t.join() for t in th]
    assert not errors, errors
    total = sum(base.astype(np.float64) * (r + 1) * steps + sum(range(1, steps + 1)) for r in range(world))
    if mode == "sync":
        assert np.array_equal(applied[0], total) and np.array_equal(applied[1], total)
    else:
        assert np.array_equal(applied[0], applied[1])               # every replica applied the same total
        assert np.all(applied[0] <= total + 1e-6) and applied[0].sum() > 0


@pytest.mark.parametrize("seed", range(24))
def test_randomised_schedules_keep_the_invariants(seed):
    """Random worlds, modes, limiters, grace windows, staleness policies and delay patterns: every rank's result is
    untorn, no wait runs out, every replica has applied the same total once the channel is flushed, nothing is
    counted twice, and with accumulation plus two closing synchronous rounds nothing is lost."""
    cfg = random.Random(1000 + seed)
    world = cfg.choice([2, 3, 4, 5, 6])
    mode = cfg.choice(["solo", "majority"])
    limiter = cfg.choice([-1, 1, 3, 8])
    accumulate = cfg.random() < 0.5
    kw = dict(seed=cfg.randrange(1 << 30), average="sum", timeout_s=30, accumulate=accumulate,
              include_stale=cfg.random() < 0.7, grace_us=cfg.choice([0.0, 200.0]), adaptive_grace=cfg.random() < 0.5)
    p_delay = [cfg.choice([0.0, 0.2, 0.6, 1.0]) for _ in range(world)]
    scale = cfg.choice([0.0005, 0.002, 0.004])
    count, steps = 32, 30
    segs = LocalSegments(world, count, np.int64)
    applied = [0] * world
    stats = [None] * world
    errors = []
    phase = threading.Barrier(world)

    def worker(r):
        try:
            ch = CpuChannel(segs.bases, r, world, count, np.int64, mode=mode, limiter=limiter, **kw)
            rng = random.Random(seed * 977 + r)
            for k in range(1, steps + 1):
                if rng.random() < p_delay[r]:
                    time.sleep(rng.random() * scale)
                out, _ = ch.step(np.full(count, (r + 1) * 1000 + k, dtype=np.int64))
                assert np.all(out == out[0]), "torn result"
                applied[r] += int(out[0])
            phase.wait()
            if accumulate:
                closing = CpuChannel(segs.bases, r, world, count, np.int64, mode="sync", limiter=-1, **kw)
                for _ in range(2):
                    out, _ = closing.step(np.zeros(count, dtype=np.int64))
                    applied[r] += int(out[0])
                stats[r] = closing.stats()
            else:
                out, _ = ch.flush()
                applied[r] += int(out[0])
                stats[r] = ch.stats()
        except Exception as e:  # noqa
            errors.append((r, repr(e)))
            try:
                phase.abort()
            except Exception:
                pass

    th = [threading.Thread(target=worker, args=(r,)) for r in range(world)]
    [t.start() for t in th]
    [t.join() for t in th]
    desc = dict(world=world, mode=mode, limiter=limiter, accumulate=accumulate, kw=kw, p_delay=p_delay, scale=scale)
    assert not errors, (errors, desc)
    published = sum((r + 1) * 1000 + k for r in range(world) for k in range(1, steps + 1))
    assert all(s["status"] == 0 for s in stats), (stats, desc)
    assert len(set(applied)) == 1, (applied, desc)                  # replicas agree
    assert applied[0] <= published, (applied[0], published, desc)    # nothing twice
    if accumulate:
        assert applied[0] == published, (applied[0], published, desc)
        assert all(s["dropped_grads"] == 0 for s in stats), (stats, desc)
