"""The shared-memory MPI subset under ``baseline/mpi_shim`` and the unmodified reference library built on it.

The reference's own correctness programs are the check: its synchronous allreduce against a closed form
(fflib2 evaluation/allreduce.c:24-44, 2048 fresh schedules), and its solo / majority allreduce against
``MPI_Allreduce`` with barriers around every round (solo_allreduce_correctness.c:76-99,
rand_allreduce_correctness.c:78-101) — which exercises the shim's point-to-point matching, its barriers
and its allreduce at once.  Skipped where the reference sources are not present.
"""
import os
import shutil
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "baseline"))
BIN = os.path.join(ROOT, "baseline", "_ref", "bin")


@pytest.fixture(scope="module")
def ref_bin():
    if shutil.which("gcc") is None:
        pytest.skip("no C compiler")
    import run_reference
    why = run_reference.available()
    if why:
        pytest.skip(why)
    return BIN


def _run(ref_bin, ranks, prog, *args, timeout=300):
    r = subprocess.run([os.path.join(ref_bin, "shimrun"), "-n", str(ranks), os.path.join(ref_bin, prog)] +
                       [str(a) for a in args], capture_output=True, text=True, timeout=timeout, cwd=ref_bin)
    return r.returncode, r.stdout + r.stderr


def test_point_to_point_and_dependencies(ref_bin):
    rc, out = _run(ref_bin, 2, "send_recv", 100000)
    assert rc == 0 and "Success!" in out, out[-500:]
    rc, out = _run(ref_bin, 2, "ping_pong_dep", 3000000, 5)      # larger than a ring: streamed in pieces
    assert rc == 0 and out.count("Success!") >= 1, out[-500:]


@pytest.mark.parametrize("ranks", [2, 4])
def test_reference_allreduce_closed_form(ref_bin, ranks):
    rc, out = _run(ref_bin, ranks, "allreduce", 1000)
    assert rc == 0 and "PASSED!" in out and "FAILED" not in out, out[-500:]


@pytest.mark.parametrize("prog", ["solo_allreduce_correctness", "rand_allreduce_correctness"])
def test_reference_partial_allreduce_against_shim_allreduce(ref_bin, prog):
    rc, out = _run(ref_bin, 4, prog, 2000, 20, 0)
    assert rc == 0 and "check passed" in out, out[-500:]


def test_sgd_loop_figures_are_parsed(ref_bin):
    import run_reference
    res = run_reference.run(ranks=(2,), counts=(1024,), iters=6)
    row = res["rows"][0]
    assert all(row[k] is not None and row[k] > 0 for k in ("ssgd_us", "rsgd_us", "randomsgd_us")), row


def test_bench_reference_arm_prints_one_json_line():
    """``bench.py --impl reference`` on any machine: one JSON line that says why the training path of the reference
    is unavailable and carries the figures of its own fflib2 loops."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2",
                        "--warmup", "1"], capture_output=True, text=True, timeout=900, cwd=root)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    rec = json.loads(lines[0])
    assert rec["impl"] == "reference" and "tensorflow" in rec["unavailable"]
    loops = rec.get("fflib2_sgd_loops", {})
    if "rows" in loops:                                   # the library was built here: its loops ran
        assert all(row["rsgd_us"] is None or row["rsgd_us"] > 0 for row in loops["rows"])
