"""ctypes bindings of the two native libraries (host control plane, CUDA kernels)."""
from __future__ import annotations

import ctypes as C

from .. import _build

MAX_RANKS = 16
MODE_SOLO, MODE_MAJORITY, MODE_SYNC = 0, 1, 2
ROLE_ABORT, ROLE_PARTICIPANT, ROLE_DRAIN, ROLE_IDLE = 0, 1, 2, 3
ROLE_NAMES = {0: "abort", 1: "participant", 2: "drain", 3: "idle"}
AVG_CONTRIBUTORS, AVG_WORLD, AVG_SUM = 0, 1, 2
DT_F32, DT_F64, DT_I32, DT_I64 = 0, 1, 2, 3

STATUS_BITS = {
    1 << 0: "timeout waiting for a round",
    1 << 1: "timeout waiting for every rank to arrive (synchronous round)",
    1 << 2: "timeout taking a mailbox lock",
    1 << 3: "timeout waiting for a round to complete",
    1 << 4: "round descriptor overwritten before it was read",
    1 << 5: "participant found data in its own mailbox",
    1 << 6: "timeout waiting for a publish slot to be released",
    1 << 7: "timeout waiting for a participant's share of the reduced vector (two-shot reduction)",
    1 << 8: "the blocks of a rank's reduce kernel did not meet at a barrier in time",
}


def status_text(status: int) -> str:
    return "; ".join(t for b, t in STATUS_BITS.items() if status & b) or "ok"


class ChannelError(RuntimeError):
    """A bounded wait of the partial allreduce ran out (a rank is missing or dead)."""

    def __init__(self, status: int, where: str = ""):
        self.status = status
        super().__init__("partial allreduce failed%s: %s" % (" (" + where + ")" if where else "", status_text(status)))


class CpuParams(C.Structure):
    _fields_ = [(n, C.c_int32) for n in
                "rank world base_mode include_stale average home dtype flags".split()] + \
               [("limiter", C.c_int64)] + \
               [(n, C.c_uint64) for n in "seed timeout_ns grace_ns count".split()]


class StepInfo(C.Structure):
    _fields_ = [("role", C.c_int32), ("n_contrib", C.c_int32), ("n_fresh", C.c_int32), ("is_sync", C.c_int32),
                ("status", C.c_uint32), ("drain_rounds", C.c_float), ("round", C.c_uint64),
                ("local_step", C.c_uint64)]


class ChannelDesc(C.Structure):
    _fields_ = [("ctl", C.c_void_p * MAX_RANKS), ("slot0", C.c_void_p * MAX_RANKS),
                ("slot1", C.c_void_p * MAX_RANKS), ("red", C.c_void_p * MAX_RANKS),
                ("rsum", C.c_void_p * MAX_RANKS)] + \
               [(n, C.c_int32) for n in
                "rank world base_mode include_stale average home slot_bf16 grad_in_bf16".split()] + \
               [("limiter", C.c_int64)] + \
               [(n, C.c_uint64) for n in "seed timeout_ns grace_ns count".split()] + \
               [(n, C.c_void_p) for n in "grad_in w32 mom w16 out".split()] + \
               [("out_bf16", C.c_int32), ("pad", C.c_int32), ("hyper", C.c_void_p), ("two_shot_min", C.c_uint64),
                ("accumulate", C.c_int32), ("adaptive_grace", C.c_int32), ("clear_grad", C.c_int32),
                ("pad3", C.c_int32), ("mc_slot0", C.c_void_p), ("mc_slot1", C.c_void_p), ("mc_red", C.c_void_p),
                ("mc_min", C.c_uint64)]


STAT_NAMES = ("local_step", "participated", "absent", "activated", "sync_rounds", "dropped_grads",
              "contrib_sum", "wait_ns", "last_round", "last_contrib", "status", "latest_round", "folded_grads")

_host = None
_cuda = None


def host():
    global _host
    if _host is None:
        lib = _build.load_host()
        lib.esgd_ctl_bytes.restype = C.c_uint64
        lib.esgd_cpu_segment_bytes.restype = C.c_uint64
        lib.esgd_cpu_segment_bytes.argtypes = [C.c_uint64, C.c_int]
        lib.esgd_cpu_segment_init.argtypes = [C.c_void_p, C.c_uint64]
        lib.esgd_cpu_step.restype = C.c_uint32
        lib.esgd_cpu_step.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        lib.esgd_cpu_flush.restype = C.c_uint32
        lib.esgd_cpu_flush.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        lib.esgd_ctl_stats.argtypes = [C.c_void_p, C.c_void_p]
        lib.esgd_ctl_clear_status.argtypes = [C.c_void_p]
        lib.esgd_ctl_trace.restype = C.c_int32
        lib.esgd_ctl_trace.argtypes = [C.c_void_p, C.c_void_p, C.c_int32]
        lib.esgd_majority_initiator.restype = C.c_int32
        lib.esgd_majority_initiator.argtypes = [C.c_uint64, C.c_uint64, C.c_int32]
        lib.esgd_limiter_is_sync.restype = C.c_int32
        lib.esgd_limiter_is_sync.argtypes = [C.c_uint64, C.c_int64]
        _host = lib
    return _host


def cuda():
    """The CUDA kernel library; raises if it cannot be built or loaded."""
    global _cuda
    if _cuda is None:
        lib = _build.load_cuda()
        lib.esgd_dev_channel_bytes.restype = C.c_uint64
        lib.esgd_dev_ctl_bytes.restype = C.c_uint64
        lib.esgd_channel_configure.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        lib.esgd_channel_step.argtypes = [C.c_void_p, C.c_uint64, C.c_int, C.c_void_p]
        lib.esgd_channel_applied.argtypes = [C.c_void_p, C.POINTER(C.c_int), C.c_void_p]
        lib.esgd_channel_times.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        lib.esgd_set_hyper.argtypes = [C.c_void_p, C.c_float, C.c_float, C.c_float, C.c_int, C.c_float, C.c_void_p]
        lib.esgd_channel_flush.argtypes = [C.c_void_p, C.c_uint64, C.c_int, C.c_void_p]
        lib.esgd_emulated_step.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        lib.esgd_spin.argtypes = [C.c_uint64, C.c_void_p]
        lib.esgd_fused_sgd.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64,
                                       C.c_float, C.c_float, C.c_float, C.c_int, C.c_float, C.c_void_p]
        lib.esgd_arena_alloc.argtypes = [C.c_uint64, C.POINTER(C.c_void_p), C.c_void_p]
        lib.esgd_arena_open.argtypes = [C.c_void_p, C.POINTER(C.c_void_p)]
        lib.esgd_arena_close.argtypes = [C.c_void_p]
        lib.esgd_arena_free.argtypes = [C.c_void_p]
        lib.esgd_enable_peer.argtypes = [C.c_int]
        lib.esgd_memcpy_d2h.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p]
        lib.esgd_launch_count.restype = C.c_uint64
        lib.esgd_cuda_error_string.restype = C.c_char_p
        lib.esgd_cuda_error_string.argtypes = [C.c_int]
        _cuda = lib
    return _cuda


def check_cuda(code: int, what: str) -> None:
    if code != 0:
        msg = cuda().esgd_cuda_error_string(code) if code > 0 else b"invalid argument"
        raise RuntimeError("%s failed: CUDA error %d (%s)" % (what, code, msg.decode()))


def parse_stats(raw) -> dict:
    d = {n: int(raw[i]) for i, n in enumerate(STAT_NAMES)}
    t = [int(raw[16 + q]) for q in range(6)]
    us = lambda a, b: (t[b] - t[a]) / 1e3 if t[a] and t[b] else None
    # newest control step: publishing, the election, the activator's waits and its descriptor broadcast, and
    # the time until the round was visible here
    d["control_us"] = {"publish": us(0, 1), "elect": us(1, 2), "activate_wait": us(2, 3), "describe": us(3, 4),
                       "visible": us(0, 5)}
    return d


def launch_count() -> int:
    """Kernels launched so far by the CUDA library of this package."""
    return int(cuda().esgd_launch_count())


TRACE_FIELDS = ("step", "round", "t_ns", "wait_ns", "role", "activator", "fresh_mask", "contrib_mask", "is_sync",
                "drain_rounds")


def parse_trace(ctl_host_ptr) -> list:
    """Trace ring of a control block that is readable from the host (CPU segment or a host copy)."""
    rows = (C.c_uint64 * (64 * 10))()
    n = host().esgd_ctl_trace(ctl_host_ptr, rows, 64)
    out = []
    for i in range(n):
        e = {f: int(rows[i * 10 + j]) for j, f in enumerate(TRACE_FIELDS)}
        e["role"] = ROLE_NAMES.get(e["role"], str(e["role"]))
        out.append(e)
    return out
