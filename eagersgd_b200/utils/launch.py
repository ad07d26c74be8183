"""Re-launch the running script as N ranks of one node.

``fork(n)`` is what the reference's ``mpi_fork`` does with ``mpiexec -np n`` (deep500/utils/mpi_helper.py:5-33):
called at the top of a script it starts ``n`` copies of that script under ``torch.distributed.run`` (one process
per rank, rendezvous on 127.0.0.1) and returns ``"parent"`` in the launching process once they have finished, or
``"child"`` inside each rank, where ``RANK`` / ``WORLD_SIZE`` / ``LOCAL_RANK`` are set.
"""
from __future__ import annotations

import os
import socket
import subprocess
import sys
from typing import List, Optional

_MARK = "EAGERSGD_FORKED"


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def fork(n: int, argv: Optional[List[str]] = None, env: Optional[dict] = None, timeout: Optional[float] = None) -> str:
    if n <= 1 or os.environ.get(_MARK) == "1" or "RANK" in os.environ:
        return "child"
    argv = list(sys.argv if argv is None else argv)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(n), "--master-addr",
           "127.0.0.1", "--master-port", str(free_port())] + argv
    child_env = dict(os.environ)
    child_env.update(env or {})
    child_env[_MARK] = "1"
    rc = subprocess.run(cmd, env=child_env, timeout=timeout).returncode
    if rc != 0:
        raise RuntimeError("%d ranks of %s ended with exit code %d" % (n, argv[0], rc))
    return "parent"


def rank_env() -> dict:
    """RANK / LOCAL_RANK / WORLD_SIZE of this process (single-process defaults when not launched as a rank)."""
    return {"rank": int(os.environ.get("RANK", 0)), "local_rank": int(os.environ.get("LOCAL_RANK", 0)),
            "world": int(os.environ.get("WORLD_SIZE", 1))}


def end_barrier() -> None:
    """Meet the other ranks once more and leave the process group, if this process is a rank of one; nothing
    otherwise.  The last line of a program that may or may not have been forked into ranks (the reference's
    ``mpi_end_barrier``, deep500/utils/mpi_helper.py:48-57)."""
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized():
        dist.barrier()
        from ..parallel.group import finalize
        finalize()
