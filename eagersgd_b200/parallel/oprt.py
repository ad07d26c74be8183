"""Python binding of the host operation runtime (``csrc/host/oprt.{h,cpp}``): persistent,
dependency-triggered operations and schedules, the programming model of the reference's fflib2
(src/ff.h:100-165).  Ranks are threads of one process; see ``World``."""
from __future__ import annotations

import ctypes as C
from typing import Callable, List, Optional, Tuple

import numpy as np

from .. import _build

INT32, INT64, FLOAT, DOUBLE, CHAR = 0, 1, 2, 3, 4
SHADOW_TAG, COMPLETE_BEFORE_CANCELLING, COMP_DEST_ATOMIC = 0x100, 0x200, 0x400
SUM, PROD, MAX, MIN, IDENTITY = 0, 1, 2, 3, 4
DEP_AND, DEP_OR, DEP_FIRST, NON_PERSISTENT = 0, 1, 2, 4
INPLACE, NONE = -2, -1
COMPLETED, SUCCESS, ERROR, TIMEOUT = 1, 0, -1, -2
_DT = {np.dtype("int8"): CHAR, np.dtype("int32"): INT32, np.dtype("int64"): INT64, np.dtype("float32"): FLOAT, np.dtype("float64"): DOUBLE}

CALLBACK = C.CFUNCTYPE(None, C.c_int64, C.c_void_p)
OPERATOR = C.CFUNCTYPE(None, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int)
SCHED_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_int64)
SCHED_WAIT_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_int64, C.c_double)
DEP_IGNORE_VERSION, DEP_NO_AUTOPOST, DEP_CONSTRAINED, DEP_SKIP_OLD_VERSIONS = 0x10, 0x20, 0x40, 0x80
PARTIAL_STALE, PARTIAL_ACCUMULATE, PARTIAL_LIVE = 0x800, 0x1000, 0x2000
NONE = -1

_lib = None


def lib():
    global _lib
    if _lib is None:
        l = C.CDLL(_build.build_host())
        vp, i64, i32 = C.c_void_p, C.c_int64, C.c_int
        l.rt_world_create.restype = vp
        l.rt_world_create.argtypes = [i32]
        l.rt_world_destroy.argtypes = [vp]
        l.rt_world_rank.restype = vp
        l.rt_world_rank.argtypes = [vp, i32]
        l.rt_buffer_create.restype = i64
        l.rt_buffer_create.argtypes = [vp, vp, i64, i32]
        l.rt_buffer_resize.argtypes = [vp, i64, vp, i64]
        l.rt_buffer_count.restype = i64
        l.rt_buffer_count.argtypes = [vp, i64]
        l.rt_buffer_data.restype = vp
        l.rt_buffer_data.argtypes = [vp, i64]
        for name, args in (("rt_op_nop", [vp, i32]), ("rt_op_callback", [vp, CALLBACK, vp, i32]),
                           ("rt_op_comp", [vp, i64, i64, i64, i32, i32]), ("rt_op_send", [vp, i64, i32, i32, i32]),
                           ("rt_op_recv", [vp, i64, i32, i32, i32]), ("rt_schedule_create", [vp]),
                           ("rt_schedule_begin_op", [vp, i64]), ("rt_schedule_end_op", [vp, i64]),
                           ("rt_allreduce", [vp, i64, i64, i32, i32]), ("rt_op_completions", [vp, i64])):
            getattr(l, name).restype = i64
            getattr(l, name).argtypes = args
        l.rt_operator_create.argtypes = [vp, OPERATOR]
        l.rt_op_hb.argtypes = [vp, i64, i64]
        l.rt_op_post.argtypes = [vp, i64]
        l.rt_op_wait.argtypes = [vp, i64, C.c_double]
        l.rt_op_test.argtypes = [vp, i64]
        l.rt_schedule_add_op.argtypes = [vp, i64, i64]
        l.rt_schedule_finalize.argtypes = [vp, i64]
        l.rt_schedule_post.argtypes = [vp, i64]
        l.rt_schedule_wait.argtypes = [vp, i64, C.c_double]
        l.rt_schedule_test.argtypes = [vp, i64]
        l.rt_schedule_print.argtypes = [vp, i64, C.c_char_p, i64]
        l.rt_schedule_print_visjs.argtypes = [vp, i64, C.c_char_p, i64]
        l.rt_buffer_delete.argtypes = [vp, i64]
        l.rt_op_hb_fallback.argtypes = [vp, i64, i64, i64, i32, C.POINTER(i64)]
        l.rt_dep_set_parent.argtypes = [vp, i64, i64]
        l.rt_op_cancel.argtypes = [vp, i64]
        l.rt_op_free.argtypes = [vp, i64]
        l.rt_schedule_start.argtypes = [vp, i64]
        l.rt_schedule_delete.argtypes = [vp, i64]
        l.rt_schedule_add_part.argtypes = [vp, i64, i64]
        l.rt_schedule_own_buffer.argtypes = [vp, i64, i64]
        for nm in ("start", "post", "test", "delete"):
            getattr(l, "rt_schedule_set_%s_fun" % nm).argtypes = [vp, i64, SCHED_FN]
        l.rt_schedule_set_wait_fun.argtypes = [vp, i64, SCHED_WAIT_FN]
        for nm in ("post", "test"):
            getattr(l, "rt_schedule_default_" + nm).argtypes = [vp, i64]
        l.rt_schedule_default_wait.argtypes = [vp, i64, C.c_double]
        l.rt_schedule_set_state.argtypes = [vp, i64, vp]
        l.rt_schedule_get_state.restype = vp
        l.rt_schedule_get_state.argtypes = [vp, i64]
        l.rt_activation.restype = i64
        l.rt_activation.argtypes = [vp, i32, C.POINTER(i64), C.POINTER(i64)]
        l.rt_limiter.argtypes = [vp, i32, C.POINTER(i64), C.POINTER(i64), C.POINTER(i64)]
        l.rt_op_tostring.argtypes = [vp, i64, C.c_char_p, i64]
        l.rt_operator_delete.argtypes = [vp, i32]
        l.rt_schedule_default_delete.argtypes = [vp, i64]
        l.rt_schedule_default_print.argtypes = [vp, i64, C.c_char_p, i64]
        l.rt_solo_allreduce.restype = i64
        l.rt_solo_allreduce.argtypes = [vp, i64, i64, i32, i32, i32, i32]
        l.rt_rand_allreduce.restype = i64
        l.rt_rand_allreduce.argtypes = [vp, i64, i64, i32, i32, i32, i32, i32]
        l.rt_partial_info.argtypes = [vp, i64, C.POINTER(i64)]
        l.rt_partial_read.argtypes = [vp, i64, vp, C.POINTER(i64), C.POINTER(i64)]
        l.rt_partial_activator.argtypes = [vp, i64, i64]
        _lib = l
    return _lib


class Rank:
    """One rank's view of the runtime (an ``rt_rank``)."""

    def __init__(self, world: "World", r: int):
        self.world, self.id, self.size = world, r, world.n
        self.h = lib().rt_world_rank(world.h, r)
        self._keep = []   # numpy arrays and callbacks referenced by the native side

    # buffers
    def buffer(self, array: Optional[np.ndarray] = None, count: int = 0, dtype=np.float32) -> int:
        if array is not None:
            self._keep.append(array)
            return lib().rt_buffer_create(self.h, array.ctypes.data, array.size, _DT[array.dtype])
        return lib().rt_buffer_create(self.h, None, count, _DT[np.dtype(dtype)])

    def resize(self, buf: int, array: Optional[np.ndarray] = None, count: int = 0):
        if array is not None:
            self._keep.append(array)
            return lib().rt_buffer_resize(self.h, buf, array.ctypes.data, array.size)
        return lib().rt_buffer_resize(self.h, buf, None, count)

    def buffer_array(self, buf: int, dtype=np.float32) -> np.ndarray:
        n = lib().rt_buffer_count(self.h, buf)
        ptr = lib().rt_buffer_data(self.h, buf)
        return np.ctypeslib.as_array(C.cast(ptr, C.POINTER(np.ctypeslib.as_ctypes_type(np.dtype(dtype)))), (n,))

    # operations
    def nop(self, options=0): return lib().rt_op_nop(self.h, options)

    def callback(self, fn: Callable[[int], None], options=0):
        cb = CALLBACK(lambda op, arg: fn(op))
        self._keep.append(cb)
        return lib().rt_op_callback(self.h, cb, None, options)

    def comp(self, a, b, out, op=SUM, options=0): return lib().rt_op_comp(self.h, a, b, out, op, options)
    def send(self, buf, peer, tag, options=0): return lib().rt_op_send(self.h, buf, peer, tag, options)
    def recv(self, buf, peer, tag, options=0): return lib().rt_op_recv(self.h, buf, peer, tag, options)

    def operator(self, fn: Callable[[np.ndarray, np.ndarray, np.ndarray], None], dtype=np.int32) -> int:
        ct = np.ctypeslib.as_ctypes_type(np.dtype(dtype))

        def tramp(a, b, o, n, dt):
            arr = lambda p: np.ctypeslib.as_array(C.cast(p, C.POINTER(ct)), (n,))
            fn(arr(a), arr(b), arr(o))
        cb = OPERATOR(tramp)
        self._keep.append(cb)
        return lib().rt_operator_create(self.h, cb)

    def operator_delete(self, oper: int): return lib().rt_operator_delete(self.h, oper)

    def describe(self, op: int) -> str:
        """One line on an operation (``ffop_tostring``)."""
        buf = C.create_string_buffer(512)
        return buf.value.decode() if lib().rt_op_tostring(self.h, op, buf, len(buf)) >= 0 else ""

    def hb(self, first, second): return lib().rt_op_hb(self.h, first, second)
    def hb_fallback(self, first, second, fallback=NONE, options=0) -> int:
        """Versioned edge (the n-th completion of ``first`` feeds the n-th run of ``second``; a completion that
        comes too late goes to ``fallback``).  Returns the edge handle."""
        d = C.c_int64()
        lib().rt_op_hb_fallback(self.h, first, second, fallback, options, C.byref(d))
        return d.value

    def dep_set_parent(self, constrained: int, constraining: int): return lib().rt_dep_set_parent(self.h, constrained, constraining)
    def cancel(self, op): return lib().rt_op_cancel(self.h, op)
    def free(self, op): return lib().rt_op_free(self.h, op)
    def buffer_delete(self, buf): return lib().rt_buffer_delete(self.h, buf)
    def post(self, op): return lib().rt_op_post(self.h, op)
    def wait(self, op, timeout=30.0): return lib().rt_op_wait(self.h, op, timeout)
    def test(self, op): return lib().rt_op_test(self.h, op)
    def completions(self, op): return lib().rt_op_completions(self.h, op)

    # schedules
    def schedule(self): return lib().rt_schedule_create(self.h)
    def schedule_add(self, s, op): return lib().rt_schedule_add_op(self.h, s, op)
    def schedule_start(self, s): return lib().rt_schedule_start(self.h, s)
    def schedule_delete(self, s): return lib().rt_schedule_delete(self.h, s)
    def schedule_add_part(self, s, part): return lib().rt_schedule_add_part(self.h, s, part)

    def schedule_override(self, s, start=None, post=None, wait=None, test=None, delete=None):
        """Replace what start / post / wait / test / delete of schedule ``s`` do (composite schedules).  The
        callables get the schedule handle (``wait`` also the timeout) and return a runtime code; the defaults
        stay reachable as ``schedule_default_post / _wait / _test``."""
        keep = self._keep
        for name, fn, proto in (("start", start, SCHED_FN), ("post", post, SCHED_FN), ("test", test, SCHED_FN),
                                ("delete", delete, SCHED_FN)):
            if fn is not None:
                cb = proto(lambda c, sid, fn=fn: int(fn(sid) or 0))
                keep.append(cb)
                getattr(lib(), "rt_schedule_set_%s_fun" % name)(self.h, s, cb)
        if wait is not None:
            cb = SCHED_WAIT_FN(lambda c, sid, t, fn=wait: int(fn(sid, t) or 0))
            keep.append(cb)
            lib().rt_schedule_set_wait_fun(self.h, s, cb)

    def schedule_default_post(self, s): return lib().rt_schedule_default_post(self.h, s)
    def schedule_default_wait(self, s, timeout=30.0): return lib().rt_schedule_default_wait(self.h, s, timeout)
    def schedule_default_test(self, s): return lib().rt_schedule_default_test(self.h, s)
    def schedule_post(self, s): return lib().rt_schedule_post(self.h, s)
    def schedule_wait(self, s, timeout=30.0): return lib().rt_schedule_wait(self.h, s, timeout)
    def schedule_test(self, s): return lib().rt_schedule_test(self.h, s)
    def schedule_end(self, s): return lib().rt_schedule_end_op(self.h, s)

    def schedule_dot(self, s) -> str:
        buf = C.create_string_buffer(1 << 16)
        n = lib().rt_schedule_print(self.h, s, buf, len(buf))
        return buf.value.decode() if n >= 0 else ""

    def schedule_visjs(self, s) -> dict:
        """The schedule as ``{"nodes": [...], "edges": [...]}`` for a vis.js network view."""
        import json
        buf = C.create_string_buffer(1 << 17)
        n = lib().rt_schedule_print_visjs(self.h, s, buf, len(buf))
        return json.loads(buf.value.decode()) if n >= 0 else {}

    # collectives
    def allreduce(self, snd: int, rcv: int, tag: int, op=SUM) -> int:
        return lib().rt_allreduce(self.h, snd, rcv, tag, op)

    def activation(self, tag: int, arm: bool = True) -> Tuple[int, int, int]:
        """(schedule, activate, joined).  With ``arm=False`` the rank does not listen yet: hang dependents on ``joined``
        first and call ``schedule_start`` then, so that an activation from a faster rank cannot pass them by."""
        a, j = C.c_int64(), C.c_int64()
        s = lib().rt_activation(self.h, tag, C.byref(a), C.byref(j))
        if arm:
            lib().rt_schedule_start(self.h, s)
        return s, a.value, j.value

    def limiter(self, num_async: int) -> Tuple[int, List[int], int]:
        st, sy = C.c_int64(), C.c_int64()
        arr = (C.c_int64 * num_async)()
        lib().rt_limiter(self.h, num_async, C.byref(st), arr, C.byref(sy))
        return st.value, list(arr), sy.value

    # partial allreduces as schedules (ffsolo_allreduce / ffrand_allreduce, fflib2 src/ff.h:161-165)
    def solo_allreduce(self, snd: int, rcv: int, tag: int, op=SUM, limiter: int = -1, options: int = 0) -> int:
        """The first rank to post round j activates it on every rank; ``limiter`` >= 0 makes every (limiter+1)-th
        round synchronous.  Drive the returned schedule with ``schedule_start / _post / _wait / _test / _delete``."""
        return lib().rt_solo_allreduce(self.h, snd, rcv, tag, op, limiter, options)

    def rand_allreduce(self, snd: int, rcv: int, tag: int, op=SUM, seed: int = 0, limiter: int = -1, options: int = 0) -> int:
        """Majority allreduce: the rank drawn for round j (the same draw on every rank) activates it."""
        return lib().rt_rand_allreduce(self.h, snd, rcv, tag, op, seed, limiter, options)

    def partial_info(self, s: int) -> dict:
        out = (C.c_int64 * 9)()
        if lib().rt_partial_info(self.h, s, out) != SUCCESS:
            raise ValueError("not a live partial allreduce")
        keys = ("posts", "rounds", "activated", "late", "sync_rounds", "contributors", "round", "overwritten", "pending")
        return dict(zip(keys, list(out)))

    def partial_read(self, s: int, out: np.ndarray) -> Tuple[int, int]:
        """Copy the newest result into ``out`` together with (fresh contributors, round number), without tearing."""
        k, r = C.c_int64(), C.c_int64()
        if lib().rt_partial_read(self.h, s, out.ctypes.data_as(C.c_void_p), C.byref(k), C.byref(r)) != SUCCESS:
            raise ValueError("not a live partial allreduce")
        return k.value, r.value

    def partial_activator(self, s: int, round_: int) -> int:
        return lib().rt_partial_activator(self.h, s, round_)


class World:
    def __init__(self, nranks: int):
        self.n = nranks
        self.h = lib().rt_world_create(nranks)
        self.ranks = [Rank(self, r) for r in range(nranks)]

    def close(self):
        if self.h:
            lib().rt_world_destroy(self.h)
            self.h = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()
