"""NVTX ranges around the phases of a training step (forward, backward, each bucket's partial allreduce, the
optimizer step), for timelines in Nsight Systems.  Off unless ``ESGD_NVTX=1``: a disabled range is a no-op
context manager, so the ranges can stay in the hot path.  Counterpart of the reference's trace builds
(fflib2 ``FFLOG`` / ``FFGRAPH``) on the profiler side; the always-on device trace ring is in the channel."""
from __future__ import annotations

import contextlib
import os

_ON = None


def nvtx_enabled() -> bool:
    global _ON
    if _ON is None:
        _ON = os.environ.get("ESGD_NVTX", "0") == "1"
    return _ON


@contextlib.contextmanager
def _range(name: str):
    import torch
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


_NULL = contextlib.nullcontext()


def nvtx_range(name: str):
    """``with nvtx_range("forward"): ...``"""
    return _range(name) if nvtx_enabled() else _NULL
