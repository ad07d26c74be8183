"""Host operation runtime: the reference's fflib2 evaluation programs as assertions
(evaluation/send_recv.c, ping_pong_dep.c, ping_pong_schedule.c, simple_computation.c,
custom_computation.c, first_dep.c, activation_1.c, activation_tree_multiple.c, limiter.c,
allreduce.c, allreduce_inplace.c, allreduce_buffers_user_managed*.c, allreduce_buffers_fflib_managed*.c,
ping_modify_pong.c, activation_tree.c).  The solo / majority programs are in test_oprt_partial.py."""
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
        except Exception as e:  # noqa
            import traceback
            errs.append(traceback.format_exc())
    th = [threading.Thread(target=wrap, args=(world.ranks[r],)) for r in range(world.n)]
    [t.start() for t in th]
    [t.join() for t in th]
    assert not errs, errs[0]


def test_send_recv():
    with R.World(2) as w:
        data = np.arange(64, dtype=np.int32)
        got = np.zeros(64, dtype=np.int32)
        r0, r1 = w.ranks
        s = r0.send(r0.buffer(data), 1, 3)
        rv = r1.recv(r1.buffer(got), 0, 3)
        r1.post(rv)
        r0.post(s)
        assert r1.wait(rv) == R.SUCCESS and r0.wait(s) == R.SUCCESS
        assert np.array_equal(got, data)


def test_ping_pong_with_dependency_is_persistent():
    """recv -> send happens-before edge; the same ops are re-posted every iteration."""
    with R.World(2) as w:
        r0, r1 = w.ranks
        ping, pong = np.zeros(8, dtype=np.int64), np.zeros(8, dtype=np.int64)
        echo = np.zeros(8, dtype=np.int64)
        s0 = r0.send(r0.buffer(ping), 1, 0)
        v0 = r0.recv(r0.buffer(pong), 1, 1)
        v1 = r1.recv(r1.buffer(echo), 0, 0)
        s1 = r1.send(r1.buffer(echo), 0, 1)
        r1.hb(v1, s1)                       # the pong is sent once the ping has arrived
        for it in range(20):
            ping[:] = it
            r1.post(v1)
            r0.post(v0)
            r0.post(s0)
            assert r0.wait(v0) == R.SUCCESS
            assert np.all(pong == it)
        assert r1.completions(s1) == 20


def test_computation_builtin_and_custom_operators():
    with R.World(1) as w:
        r = w.ranks[0]
        a, b, c = np.arange(10, dtype=np.int32), np.arange(10, dtype=np.int32) * 2, np.zeros(10, dtype=np.int32)
        ba, bb, bc = r.buffer(a), r.buffer(b), r.buffer(c)
        for op, expect in ((R.SUM, a + b), (R.PROD, a * b), (R.MAX, np.maximum(a, b)), (R.MIN, np.minimum(a, b))):
            o = r.comp(ba, bb, bc, op)
            r.post(o)
            r.wait(o)
            assert np.array_equal(c, expect)
        plus_one = r.operator(lambda x, y, out: np.copyto(out, x + y + 1), np.int32)
        o = r.comp(ba, bb, bc, plus_one)
        r.post(o)
        r.wait(o)
        assert np.array_equal(c, a + b + 1)


def test_first_dependency_vs_and_fanout():
    """DEP_FIRST satisfies one dependent per completion; a plain op satisfies all of them."""
    deps = 5
    with R.World(1) as w:
        r = w.ranks[0]
        acc = {"first": 0, "all": 0}
        first = r.nop(R.DEP_FIRST)
        plain = r.nop()
        for _ in range(deps):
            r.hb(first, r.callback(lambda op: acc.__setitem__("first", acc["first"] + 1), R.DEP_OR))
            r.hb(plain, r.callback(lambda op: acc.__setitem__("all", acc["all"] + 1), R.DEP_OR))
        done = r.nop()
        for _ in range(deps):
            r.post(first)
            r.wait(first)
            r.post(plain)
            r.wait(plain)
        r.post(done)
        r.wait(done)
        import time
        time.sleep(0.05)
        assert acc["first"] == deps and acc["all"] == deps * deps


def test_or_dependency():
    n = 50
    with R.World(1) as w:
        r = w.ranks[0]
        count = [0]
        a, b = r.nop(), r.nop()
        either = r.callback(lambda op: count.__setitem__(0, count[0] + 1), R.DEP_OR)
        r.hb(a, either)
        r.hb(b, either)
        for i in range(n):
            r.post(a if i % 2 else b)
            r.wait(either)
        assert count[0] == n


def test_schedule_and_dot():
    with R.World(1) as w:
        r = w.ranks[0]
        x = np.ones(4, dtype=np.float32)
        y = np.zeros(4, dtype=np.float32)
        bx, by = r.buffer(x), r.buffer(y)
        s = r.schedule()
        c1 = r.comp(bx, bx, by, R.SUM)          # y = 2
        c2 = r.comp(by, bx, by, R.SUM)          # y = 3
        r.hb(c1, c2)
        r.schedule_add(s, c1)
        r.schedule_add(s, c2)
        for _ in range(3):
            r.schedule_post(s)
            assert r.schedule_wait(s) == R.SUCCESS
            assert np.all(y == 3)
        dot = r.schedule_dot(s)
        assert dot.startswith("digraph") and "->" in dot and "begin" in dot
        vis = r.schedule_visjs(s)                 # the same graph for a vis.js network view
        labels = sorted(n["label"] for n in vis["nodes"])
        assert labels == ["comp", "comp", "nop begin", "nop end"]
        ids = {n["id"] for n in vis["nodes"]}
        assert len(vis["edges"]) == dot.count("->") and all(e["from"] in ids and e["to"] in ids for e in vis["edges"])


@pytest.mark.parametrize("world", [1, 2, 3, 4, 5, 8])
def test_allreduce_closed_form_persistent_and_resized(world):
    """(i + j) * size closed form; the schedule is re-posted with new data and a resized buffer."""
    with R.World(world) as w:
        def body(r):
            n = 33
            snd, rcv = np.zeros(n, dtype=np.int32), np.zeros(n, dtype=np.int32)
            bs, br = r.buffer(snd), r.buffer(rcv)
            s = r.allreduce(bs, br, tag=7)
            for it in range(10):
                snd[:] = np.arange(n) + it + r.id
                r.schedule_post(s)
                assert r.schedule_wait(s) == R.SUCCESS
                expect = (np.arange(n) + it) * world + sum(range(world))
                assert np.array_equal(rcv, expect), (r.id, it, rcv[:4], expect[:4])
            # in place, float, maximum
            x = np.full(5, float(r.id), dtype=np.float64)
            bx = r.buffer(x)
            s2 = r.allreduce(R.INPLACE, bx, tag=9, op=R.MAX)
            r.schedule_post(s2)
            r.schedule_wait(s2)
            assert np.all(x == world - 1)
        _run(w, body)


def test_allreduce_completion_callback():
    with R.World(2) as w:
        fired = [0, 0]

        def body(r):
            x = np.full(4, r.id + 1, dtype=np.int64)
            s = r.allreduce(R.INPLACE, r.buffer(x), tag=1)
            cb = r.callback(lambda op: fired.__setitem__(r.id, fired[r.id] + 1), R.DEP_OR)
            r.hb(r.schedule_end(s), cb)
            r.schedule_post(s)
            r.wait(cb)
            assert np.all(x == 3)
        _run(w, body)
        assert fired == [1, 1]


def test_activation_from_random_ranks():
    """Any rank may activate; every rank's join op completes exactly once per activation."""
    world, n = 4, 30
    rng = np.random.RandomState(439634)
    activators = rng.randint(world, size=n)
    with R.World(world) as w:
        def body(r):
            s, act, joined = r.activation(tag=5)
            for k in range(n):
                if activators[k] == r.id:
                    r.post(act)
                assert r.wait(joined) == R.SUCCESS
            assert r.completions(joined) == n
        _run(w, body)


def test_limiter_pattern():
    """15 posts with 3 async slots: A A A S A A A S ... (evaluation/limiter.c prints this)."""
    with R.World(1) as w:
        r = w.ranks[0]
        start, asyncs, sync = r.limiter(3)
        seq = []
        for a in asyncs:
            r.hb(a, r.callback(lambda op: seq.append("A"), R.DEP_OR))
        end = r.callback(lambda op: seq.append("S"), R.DEP_OR)
        r.hb(sync, end)
        for _ in range(15):
            r.post(start)
            r.wait(start)
        import time
        time.sleep(0.1)
        assert "".join(seq) == "AAAS" * 3 + "AAA"


def test_wait_timeout_reports_instead_of_hanging():
    with R.World(2) as w:
        r0 = w.ranks[0]
        rv = r0.recv(r0.buffer(count=4, dtype=np.int32), 1, 99)
        r0.post(rv)
        assert r0.wait(rv, timeout=0.2) == R.TIMEOUT


def test_runtime_microbenchmark_reports_three_phases():
    from eagersgd_b200.parallel.bench_oprt import run
    r = run(ranks=3, count=256, iters=10)
    assert r["correct"] and r["create_us"] > 0 and r["execute_us"] > 0 and r["delete_us"] >= 0


def test_native_microbenchmark_checks_its_results():
    """Native threads as ranks: persistent reposts and fresh create / post / wait / delete cycles, both checked
    against the closed form inside the loop."""
    from eagersgd_b200.parallel.bench_oprt import run_native
    r = run_native(ranks=3, count=257, iters=40)
    assert r["correct"] and 0 < r["persistent_us"] < 1e5 and 0 < r["fresh_us"] < 1e5


@pytest.mark.parametrize("world", [2, 3, 5, 8])
def test_activation_stress_300_rounds(world):
    """The reference loops its activation test 300 times from a shell script (evaluation/test_activation.sh);
    here 300 activations from shared-seed random ranks run back to back on one persistent schedule."""
    n = 300
    rng = np.random.RandomState(1000 + world)
    activators = rng.randint(world, size=n)
    with R.World(world) as w:
        def body(r):
            s, act, joined = r.activation(tag=9)
            for k in range(n):
                if activators[k] == r.id:
                    r.post(act)
                assert r.wait(joined, timeout=60.0) == R.SUCCESS
            assert r.completions(joined) == n
        _run(w, body)


# ---- life cycle, cancelling, versioned edges, overridable schedules -------------------------------------------
def _rss_kb():
    with open("/proc/self/status") as f:
        for line in f:
            if line.startswith("VmRSS"):
                return int(line.split()[1])
    return 0


def test_create_and_delete_2048_schedules_keeps_memory_flat():
    """A fresh allreduce schedule per iteration, deleted after use, 2048 times
    (fflib2 evaluation/allreduce.c:24-44): handles are recycled and memory does not grow."""
    world, count, iters = 4, 256, 2048
    with R.World(world) as w:
        errors, handles = [], [set() for _ in range(world)]

        def body(r):
            rk = w.ranks[r]
            snd = np.zeros(count, dtype=np.int32)
            rcv = np.zeros(count, dtype=np.int32)
            bs, br = rk.buffer(snd), rk.buffer(rcv)
            for it in range(iters):
                snd[:] = np.arange(count) + it
                s = rk.allreduce(bs, br, 7, R.SUM)
                handles[r].add(s)
                rk.schedule_post(s)
                if rk.schedule_wait(s, 30.0) != R.SUCCESS:
                    errors.append((r, it, "timeout"))
                    return
                if not np.array_equal(rcv, (np.arange(count) + it) * world):
                    errors.append((r, it, "wrong sum"))
                    return
                assert rk.schedule_delete(s) == R.SUCCESS
                if it == 200 and r == 0:
                    body.rss0 = _rss_kb()
        body.rss0 = 0
        th = [threading.Thread(target=body, args=(r,)) for r in range(world)]
        [t.start() for t in th]
        [t.join() for t in th]
        assert not errors, errors[:3]
        assert all(len(h) <= 2 for h in handles)           # the same few schedule handles over and over
        assert _rss_kb() - body.rss0 < 20000                # < 20 MB over 1800 more create / delete cycles


def test_free_and_cancel():
    with R.World(1) as w:
        rk = w.ranks[0]
        hits = []
        a = rk.nop()
        b = rk.callback(lambda op: hits.append("b"))
        c = rk.callback(lambda op: hits.append("c"))
        rk.hb(a, b)
        rk.hb(a, c)
        rk.post(a)
        assert rk.wait(c, 5.0) == R.SUCCESS and rk.wait(b, 5.0) == R.SUCCESS
        assert rk.free(b) == R.SUCCESS                      # a's edge to b is unlinked
        rk.post(a)
        assert rk.wait(c, 5.0) == R.SUCCESS
        assert sorted(hits) == ["b", "c", "c"]
        d = rk.nop()                                        # the freed handle is handed out again
        assert d == b
        # a receive that nobody answers is withdrawn; a later wait times out instead of completing
        buf = rk.buffer(count=4, dtype=np.int32)
        rv = rk.recv(buf, 0, 99)
        rk.post(rv)
        time.sleep(0.05)
        assert rk.cancel(rv) == R.SUCCESS
        assert rk.wait(rv, 0.2) == R.TIMEOUT
        assert rk.free(rv) == R.SUCCESS and rk.free(rv) != R.SUCCESS


def test_versioned_edge_routes_late_completions_to_the_fallback():
    """The n-th completion of the first op feeds the n-th run of the second; if the second has already run
    for that version (it was posted by hand meanwhile) the completion goes to the fallback, and a completion
    that is ahead of the second op is remembered until the op gets there (fflib2 src/ffop.c:331-373)."""
    with R.World(1) as w:
        rk = w.ranks[0]
        log = []
        first = rk.nop()
        second = rk.callback(lambda op: log.append("second"))
        fb = rk.callback(lambda op: log.append("fallback"))
        rk.hb_fallback(first, second, fb, 0)
        rk.post(fb)                                         # the fallback keeps step with the versions too
        assert rk.wait(fb, 5.0) == R.SUCCESS
        log.clear()
        rk.post(first)                                      # version 1 -> second runs (its version 1)
        assert rk.wait(second, 5.0) == R.SUCCESS
        rk.post(second)                                     # second runs version 2 by hand ...
        assert rk.wait(second, 5.0) == R.SUCCESS
        rk.post(first)                                      # ... so first's version 2 is late: fallback
        assert rk.wait(fb, 5.0) == R.SUCCESS
        assert log == ["second", "second", "fallback"]
        # ahead of the dependent: first completes versions 3 and 4 while the dependent of a second edge is at 0
        log.clear()
        src = rk.nop()
        dst = rk.callback(lambda op: log.append("dst"))
        rk.post(src)
        rk.post(src)
        time.sleep(0.05)
        rk.hb_fallback(src, dst, R.NONE, 0)
        rk.post(src)                                        # version 3 > dst's version + 1: remembered
        time.sleep(0.1)
        assert log == []
        rk.post(dst)                                        # dst catches up (version 1) ...
        assert rk.wait(dst, 5.0) == R.SUCCESS
        time.sleep(0.1)
        assert log.count("dst") >= 1


def test_no_autopost_and_constrained_edges():
    with R.World(1) as w:
        rk = w.ranks[0]
        log = []
        a = rk.nop()
        b = rk.callback(lambda op: log.append("b"))
        rk.hb_fallback(a, b, R.NONE, R.DEP_IGNORE_VERSION | R.DEP_NO_AUTOPOST)
        rk.post(a)
        time.sleep(0.1)
        assert log == []                                    # the edge never posts b by itself
        # constrained: gate -> x passes a completion on only after key -> y has
        key, gate = rk.nop(), rk.nop()
        x = rk.callback(lambda op: log.append("x"))
        y = rk.callback(lambda op: log.append("y"))
        e_gate = rk.hb_fallback(gate, x, R.NONE, R.DEP_IGNORE_VERSION)
        e_key = rk.hb_fallback(key, y, R.NONE, R.DEP_IGNORE_VERSION)
        rk.dep_set_parent(e_gate, e_key)
        rk.post(gate)
        time.sleep(0.1)
        assert "x" not in log
        rk.post(key)
        assert rk.wait(y, 5.0) == R.SUCCESS
        rk.post(gate)
        assert rk.wait(x, 5.0) == R.SUCCESS


def test_overridden_schedule_functions_make_a_composite_schedule():
    """A schedule whose post / wait are replaced and which owns two part schedules, the way the reference's
    solo allreduce is one schedule over an activation, two allreduces and a limiter
    (fflib2 src/colls/ffsolo_allreduce.c:88-148)."""
    with R.World(1) as w:
        rk = w.ranks[0]
        log = []
        part_a, part_b = rk.schedule(), rk.schedule()
        rk.schedule_add(part_a, rk.callback(lambda op: log.append("a")))
        rk.schedule_add(part_b, rk.callback(lambda op: log.append("b")))
        top = rk.schedule()
        rk.schedule_add_part(top, part_a)
        rk.schedule_add_part(top, part_b)

        def post(s):
            log.append("post")
            rk.schedule_post(part_a)
            return rk.schedule_post(part_b)

        def wait(s, timeout):
            rc = rk.schedule_wait(part_a, timeout)
            return rc if rc != R.SUCCESS else rk.schedule_wait(part_b, timeout)

        rk.schedule_override(top, post=post, wait=wait, start=lambda s: log.append("start") or 0)
        assert rk.schedule_start(top) == R.SUCCESS
        for _ in range(3):
            assert rk.schedule_post(top) == R.SUCCESS
            assert rk.schedule_wait(top, 5.0) == R.SUCCESS
        assert log[0] == "start" and log.count("post") == 3 and log.count("a") == 3 and log.count("b") == 3
        assert rk.schedule_delete(top) == R.SUCCESS          # takes the parts with it
        assert rk.schedule_delete(part_a) != R.SUCCESS


def test_wait_without_timeout_is_still_bounded():
    """timeout <= 0 means the runtime's default bound, not forever (checked through the code path: a
    completed op returns at once)."""
    with R.World(1) as w:
        rk = w.ranks[0]
        a = rk.nop()
        rk.post(a)
        assert rk.wait(a, 0.0) == R.SUCCESS


def test_shadow_tags_char_buffers_and_complete_before_cancelling():
    """A shadow-tagged message never matches a receive with the plain tag of the same number; int8 buffers
    reduce; an operation created with COMPLETE_BEFORE_CANCELLING finishes what was posted when cancelled."""
    with R.World(2) as w:
        a, b = w.ranks
        data = np.array([1, 2, 3, 4], dtype=np.int8)
        ctrl = np.array([9, 9, 9, 9], dtype=np.int8)
        got_data, got_ctrl = np.zeros(4, np.int8), np.zeros(4, np.int8)
        a.post(a.send(a.buffer(ctrl), 1, 5, R.SHADOW_TAG))       # control token first, same tag number
        a.post(a.send(a.buffer(data), 1, 5))
        r_data = b.recv(b.buffer(got_data), 0, 5)
        r_ctrl = b.recv(b.buffer(got_ctrl), 0, 5, R.SHADOW_TAG)
        b.post(r_data)
        b.post(r_ctrl)
        assert b.wait(r_data, 5.0) == R.SUCCESS and b.wait(r_ctrl, 5.0) == R.SUCCESS
        assert got_data.tolist() == [1, 2, 3, 4] and got_ctrl.tolist() == [9, 9, 9, 9]
        x, y, z = np.array([1, -2, 3], np.int8), np.array([10, 20, 30], np.int8), np.zeros(3, np.int8)
        c = a.comp(a.buffer(x), a.buffer(y), a.buffer(z), R.SUM, R.COMP_DEST_ATOMIC)
        a.post(c)
        assert a.wait(c, 5.0) == R.SUCCESS and z.tolist() == [11, 18, 33]
        hits = []
        keep = a.callback(lambda op: hits.append(1), R.COMPLETE_BEFORE_CANCELLING)
        a.post(keep)
        a.cancel(keep)
        assert a.wait(keep, 5.0) == R.SUCCESS and hits == [1]


@pytest.mark.parametrize("seed", range(12))
def test_random_dependency_graphs_compute_in_dependency_order(seed):
    """Random DAGs of compute operations (each adds the results of two earlier nodes, edges as happens-before
    relations) inside one schedule, posted several times with new leaf values: every node ends up with the value a
    topological evaluation gives, on every post — a node that ran before one of its parents would not."""
    rng = np.random.RandomState(seed)
    n_leaf, n_node = 3, int(rng.randint(5, 40))
    with R.World(1) as w:
        r = w.ranks[0]
        arrays = [np.zeros(4, dtype=np.int64) for _ in range(n_leaf + n_node)]
        bufs = [r.buffer(a) for a in arrays]
        s = r.schedule()
        ops, parents = {}, {}
        for i in range(n_leaf, n_leaf + n_node):
            a, b = (int(v) for v in rng.randint(0, i, size=2))
            parents[i] = (a, b)
            ops[i] = r.comp(bufs[a], bufs[b], bufs[i], R.SUM)
            for p in (a, b):
                if p in ops:
                    r.hb(ops[p], ops[i])
            r.schedule_add(s, ops[i])
        for rep in range(3):
            for k in range(n_leaf):
                arrays[k][:] = rng.randint(-5, 6, size=4)
            for i in range(n_leaf, n_leaf + n_node):
                arrays[i][:] = -999                                  # stale values must not survive
            want = [a.copy() for a in arrays[:n_leaf]]
            for i in range(n_leaf, n_leaf + n_node):
                want.append(want[parents[i][0]] + want[parents[i][1]])
            r.schedule_post(s)
            assert r.schedule_wait(s, timeout=20.0) == R.SUCCESS
            for i in range(n_leaf, n_leaf + n_node):
                assert np.array_equal(arrays[i], want[i]), (seed, rep, i, parents[i])


def test_operation_description_operator_delete_and_default_schedule_functions():
    """ffop_tostring, ffcomp_operator_delete, ffschedule_default_delete / _print (fflib2 src/ff.h:112-159)."""
    with R.World(2) as w:
        r = w.ranks[0]
        x = np.arange(4, dtype=np.int32)
        bx = r.buffer(x)
        sd = r.send(bx, 1, 9, R.SHADOW_TAG)
        rv = r.recv(bx, 1, 4, R.DEP_OR)
        assert r.describe(sd).startswith("[%d.0] send to 1 tag 9 (shadow) deps and posted 0" % sd)
        r.post(rv)
        for _ in range(200):
            if "listening" in r.describe(rv):
                break
            time.sleep(0.001)
        assert "recv from 1 tag 4 deps or posted 1 started 1 completed 0" in r.describe(rv) and r.describe(rv).endswith("listening")
        assert r.describe(10 ** 6) == ""
        # a deleted operator's number is handed out again; a compute op that still names a deleted one does nothing
        first = r.operator(lambda a, b, o: np.copyto(o, a - b))
        second = r.operator(lambda a, b, o: np.copyto(o, a * b + 1))
        assert second == first + 1
        y, z = np.full(4, 10, dtype=np.int32), np.zeros(4, dtype=np.int32)
        by, bz = r.buffer(y), r.buffer(z)
        c1 = r.comp(by, bx, bz, first)
        r.post(c1)
        assert r.wait(c1) == R.SUCCESS and z.tolist() == [10, 9, 8, 7]
        assert "comp operator %d" % first in r.describe(c1) and "completed 1" in r.describe(c1)
        assert r.operator_delete(first) == R.SUCCESS and r.operator_delete(first) == R.ERROR
        z[:] = -1
        r.post(c1)
        assert r.wait(c1) == R.SUCCESS and z.tolist() == [-1] * 4
        assert r.operator(lambda a, b, o: np.copyto(o, a + b)) == first
        r.post(c1)
        assert r.wait(c1) == R.SUCCESS and z.tolist() == [10, 11, 12, 13]
        # an overriding delete / print reaches the schedule's own part through the default functions
        s = r.schedule()
        r.schedule_add(s, r.nop())
        calls = []

        def my_delete(sched):
            calls.append("delete")
            return R.lib().rt_schedule_default_delete(r.h, sched)
        r.schedule_override(s, delete=my_delete)
        import ctypes as C
        buf = C.create_string_buffer(4096)
        assert R.lib().rt_schedule_default_print(r.h, s, buf, len(buf)) > 0 and b"digraph" in buf.value
        assert r.schedule_delete(s) == R.SUCCESS and calls == ["delete"]
        assert r.schedule_delete(s) == R.ERROR


def test_ping_modify_pong_a_dependent_operation_needs_no_post():
    """evaluation/ping_modify_pong.c: rank 1's send hangs off its receive, so only the receive is posted; the pong
    carries what the ping brought."""
    n = 257
    with R.World(2) as w:
        def body(r):
            ping, pong = np.zeros(n, dtype=np.int32), np.zeros(n, dtype=np.int32)
            if r.id == 0:
                ping[:] = np.arange(n)
                a, b = r.send(r.buffer(ping), 1, 0), r.recv(r.buffer(pong), 1, 0)
                r.post(a)
                r.post(b)
                assert r.wait(b) == R.SUCCESS and np.array_equal(pong, np.arange(n))
            else:
                bp = r.buffer(ping)
                a, b = r.recv(bp, 0, 0), r.send(bp, 0, 0)
                r.hb(a, b)
                r.post(a)                                       # b is never posted by hand
                assert r.wait(b) == R.SUCCESS and np.array_equal(ping, np.arange(n))
            for op in (a, b):
                assert r.free(op) == R.SUCCESS
        _run(w, body)


@pytest.mark.parametrize("inplace", [False, True])
def test_allreduce_on_buffers_the_runtime_owns(inplace):
    """evaluation/allreduce_buffers_fflib_managed.c and _inplace.c: buffers created without user memory, resized to a
    random count before every post, filled and read through the runtime's own pointer; closed form (i + j) * size."""
    world, rounds = 3, 12
    counts = np.random.RandomState(7).randint(1, 300, size=rounds)
    with R.World(world) as w:
        def body(r):
            rcv = r.buffer(count=300, dtype=np.float32)
            snd = R.INPLACE if inplace else r.buffer(count=300, dtype=np.float32)
            s = r.allreduce(snd, rcv, tag=0)
            for i, count in enumerate(int(c) for c in counts):
                r.resize(rcv, count=count)
                if not inplace:
                    r.resize(snd, count=count)
                src = r.buffer_array(rcv if inplace else snd, np.float32)
                assert src.shape == (count,)
                src[:] = np.arange(count) + i
                assert r.schedule_post(s) == R.SUCCESS and r.schedule_wait(s) == R.SUCCESS
                assert np.array_equal(r.buffer_array(rcv, np.float32), (np.arange(count) + i) * world), (r.id, i)
            assert r.schedule_delete(s) == R.SUCCESS and r.buffer_delete(rcv) == R.SUCCESS
        _run(w, body)


def test_activation_feeds_a_computation_on_every_rank():
    """evaluation/activation_tree.c: a compute operation (acc += 1) hangs off the activation's join; whoever the
    activator is, every rank's accumulator goes up by exactly one per activation."""
    world = 5
    activators = np.random.RandomState(4535).randint(world, size=6)
    with R.World(world) as w:
        def body(r):
            acc, inc = np.zeros(1, dtype=np.int32), np.ones(1, dtype=np.int32)
            ba, bi = r.buffer(acc), r.buffer(inc)
            s, act, joined = r.activation(tag=0, arm=False)
            add = r.comp(ba, bi, ba, R.SUM)
            r.hb(joined, add)
            assert r.schedule_post(s) == R.SUCCESS                  # listen only now that the dependent is wired
            for k, who in enumerate(activators):
                if who == r.id:
                    r.post(act)
                assert r.wait(add) == R.SUCCESS and acc[0] >= k + 1    # the next activator may be ahead already
            gate.wait()
            assert acc[0] == len(activators) and r.completions(add) == len(activators)
        gate = threading.Barrier(world)
        _run(w, body)


def test_handles_that_were_never_given_out_are_refused():
    """Every entry point checks the handles it is given: a stale or made-up one gets RT_ERROR (or a null pointer),
    never an out-of-range index."""
    import ctypes as C
    with R.World(2) as w:
        r, L = w.ranks[0], R.lib()
        x = np.zeros(4, dtype=np.int32)
        b = r.buffer(x)
        assert L.rt_buffer_count(r.h, 99) == R.ERROR and L.rt_buffer_data(r.h, -5) is None
        assert L.rt_buffer_resize(r.h, 99, None, 4) == R.ERROR and r.buffer_delete(99) == R.ERROR
        assert r.send(99, 1, 0) == R.ERROR and r.recv(b, 7, 0) == R.ERROR and r.recv(b, -1, 0) == R.ERROR
        assert r.comp(b, 99, b) == R.ERROR and r.comp(b, b, b, R.CUSTOM0 + 3 if hasattr(R, "CUSTOM0") else 19) == R.ERROR
        assert r.comp(b, R.NONE, b, R.IDENTITY) >= 0                   # the second input of a copy may be absent
        assert r.allreduce(99, b, 0) == R.ERROR and r.allreduce(R.INPLACE, 99, 0) == R.ERROR
        assert r.solo_allreduce(b, 99, 0) == R.ERROR
        for bad in (-1, 10 ** 6):
            assert r.post(bad) == R.ERROR and r.wait(bad, 0.1) == R.ERROR and r.test(bad) == R.ERROR
            assert r.completions(bad) == R.ERROR and r.cancel(bad) == R.ERROR and r.free(bad) == R.ERROR
            assert r.schedule_post(bad) == R.ERROR and r.schedule_wait(bad, 0.1) == R.ERROR and r.schedule_test(bad) == R.ERROR
            assert r.schedule_start(bad) == R.ERROR and r.schedule_delete(bad) == R.ERROR and r.schedule_end(bad) == R.NONE
            assert r.schedule_dot(bad) == "" and r.schedule_visjs(bad) == {}
        s = r.schedule()
        n = r.nop()
        assert r.schedule_add(s, 10 ** 6) == R.ERROR and r.schedule_add(s, n) == R.SUCCESS
        assert r.schedule_add_part(s, s) == R.ERROR and r.schedule_add_part(s, 123) == R.ERROR
        assert r.free(n) == R.SUCCESS and r.post(n) == R.ERROR and r.wait(n, 0.1) == R.ERROR       # freed: stale
        assert r.schedule_delete(s) == R.SUCCESS and r.schedule_post(s) == R.ERROR
