"""Run the reference's own SGD-loop timing programs (fflib2 evaluation/ssgd.c, rsgd.c, randomsgd.c),
built unmodified by ``build_reference.py``, as host ranks of one machine, and collect what they print.

    python baseline/run_reference.py [--ranks 2,4,8] [--counts 1024,262144,6553600] [--iters 12]

Each program skews its ranks by ``usleep(rank * 1 ms)`` per iteration, times one collective on a float
vector of ``count`` elements and prints the mean over ranks of that latency per iteration
(ssgd.c:63-97: ``MPI_Allreduce``, here the shared-memory one of ``baseline/mpi_shim``; rsgd.c:77-113:
``ffsolo_allreduce``; randomsgd.c:78-113: ``ffrand_allreduce``).  This script reports, per program, rank
count and vector size, the mean of those per-iteration figures after two warm-up iterations, in
microseconds.  The transport under the library is the shim's shared-memory rings (two copies per
message), not a tuned MPI: read the figures as "the reference's algorithm and progress engine on this
host", not as what Cray MPI gave it.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
BIN = os.path.join(HERE, "_ref", "bin")
PROGRAMS = {"ssgd": "shim MPI_Allreduce (synchronous)", "rsgd": "fflib2 solo allreduce",
            "randomsgd": "fflib2 majority allreduce"}
LINE = re.compile(r"iter=(\d+), count=\d+, average runtime=([0-9.eE+-]+)")


def available() -> str:
    """'' when the binaries are there (building them from the copied sources if need be), else the reason."""
    need = [os.path.join(BIN, p) for p in list(PROGRAMS) + ["shimrun", "libfflib.so"]]
    if all(os.path.exists(p) for p in need):
        return ""
    try:
        sys.path.insert(0, HERE)
        import build_reference
        build_reference.build()
    except Exception as e:  # noqa
        return "fflib2 could not be built here: %s" % str(e).splitlines()[0][:200]
    return "" if all(os.path.exists(p) for p in need) else "fflib2 build produced no binaries"


def run_one(program: str, ranks: int, count: int, iters: int, timeout: float = 300.0):
    r = subprocess.run([os.path.join(BIN, "shimrun"), "-n", str(ranks), os.path.join(BIN, program), str(count),
                        str(iters)], capture_output=True, text=True, timeout=timeout, cwd=BIN)
    vals = [float(m.group(2)) for m in LINE.finditer(r.stdout) if int(m.group(1)) >= 2]
    if r.returncode != 0 or not vals:
        return None
    return 1e6 * sum(vals) / len(vals)


def allreduce_cycle_us(ranks: int, count: int = 1024, timeout: float = 90.0):
    """Microseconds per create + post + wait + delete of a synchronous allreduce schedule: wall time of the
    reference's evaluation/allreduce.c (2048 fresh schedules on int32 vectors, checked against the closed form)
    divided by 2048.  Includes the start of the processes (about 10 ms, i.e. 5 us per cycle)."""
    import time
    t0 = time.perf_counter()
    try:
        r = subprocess.run([os.path.join(BIN, "shimrun"), "-n", str(ranks), os.path.join(BIN, "allreduce"), str(count)],
                           capture_output=True, text=True, timeout=timeout, cwd=BIN)
    except subprocess.TimeoutExpired:
        return None
    dt = time.perf_counter() - t0
    return 1e6 * dt / 2048 if r.returncode == 0 and "PASSED" in r.stdout else None


def run(ranks=(2, 4, 8), counts=(1024, 262144, 6553600), iters: int = 12) -> dict:
    why = available()
    if why:
        return {"unavailable": why}
    rows = []
    for p in ranks:
        for c in counts:
            row = {"ranks": p, "floats": c, "bytes": 4 * c, "skew": "usleep(rank * 1 ms) per iteration"}
            for prog in PROGRAMS:
                try:
                    row[prog + "_us"] = run_one(prog, p, c, iters)
                except subprocess.TimeoutExpired:
                    row[prog + "_us"] = None
            rows.append(row)
    cycles = {}
    if os.path.exists(os.path.join(BIN, "allreduce")):
        for p in ranks:
            if p <= (os.cpu_count() or 1):
                cycles[str(p)] = allreduce_cycle_us(p)
    return {"programs": PROGRAMS, "iters": iters, "transport": "shared-memory MPI subset (baseline/mpi_shim)",
            "rows": rows, "allreduce_schedule_cycle_us": cycles}


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ranks", default="2,4,8")
    ap.add_argument("--counts", default="1024,262144,6553600")
    ap.add_argument("--iters", type=int, default=12)
    a = ap.parse_args()
    print(json.dumps(run([int(x) for x in a.ranks.split(",")], [int(x) for x in a.counts.split(",")], a.iters)))
