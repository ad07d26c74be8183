"""Build the reference's communication library (fflib2) and its evaluation programs, unmodified,
against the shared-memory MPI subset in ``baseline/mpi_shim``.

    python baseline/build_reference.py [--source /path/to/eager-SGD-modules/fflib2]

The sources are copied verbatim into ``baseline/_ref/fflib2`` (the reference tree is read-only and the
build writes next to them) and compiled with the flags of the reference's own build
(fflib2 CMakeLists.txt:80-81: ``-O3 -ftree-vectorize``; evaluation/CMakeLists.txt builds one
executable per program and links ``fflib``).  Results: ``baseline/_ref/bin/libfflib.so``, ``shimrun``
and one executable per evaluation program.  Nothing in the framework links against any of this.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
SHIM = os.path.join(HERE, "mpi_shim")
# where the reference's fflib2 sources are: ESGD_REFERENCE_FFLIB2, else a checkout named "reference" beside this repository
DEFAULT_SOURCE = os.environ.get("ESGD_REFERENCE_FFLIB2") or os.path.join(
    os.path.dirname(os.path.dirname(HERE)), "reference", "eager-SGD-modules", "fflib2")
# the programs the comparison uses, plus the correctness programs that double as a check of the shim
PROGRAMS = ["ssgd", "rsgd", "randomsgd", "allreduce", "allreduce_inplace", "solo_allreduce_correctness",
            "rand_allreduce_correctness", "activation_tree_multiple", "send_recv", "ping_pong_dep", "first_dep",
            "limiter", "custom_computation", "solo_allreduce_multiple"]


def run(cmd, **kw):
    r = subprocess.run(cmd, capture_output=True, text=True, **kw)
    if r.returncode != 0:
        raise RuntimeError("%s\n%s" % (" ".join(cmd), (r.stdout + r.stderr)[-3000:]))
    return r


def build(source: str = DEFAULT_SOURCE, force: bool = False) -> str:
    src_dst = os.path.join(REF, "fflib2")
    bin_dir = os.path.join(REF, "bin")
    if os.path.isdir(source) and (force or not os.path.isdir(src_dst)):
        if os.path.isdir(src_dst):
            shutil.rmtree(src_dst)
        shutil.copytree(source, src_dst)
    if not os.path.isdir(src_dst):
        raise RuntimeError("no fflib2 sources: neither %s nor %s exists" % (source, src_dst))
    os.makedirs(bin_dir, exist_ok=True)
    cc = os.environ.get("CC", "gcc")
    inc = ["-I", SHIM, "-I", os.path.join(src_dst, "src")]
    lib_sources = []
    for root, _, files in os.walk(os.path.join(src_dst, "src")):
        lib_sources += [os.path.join(root, f) for f in files if f.endswith(".c")]
    lib_sources.sort()
    common = ["-O3", "-ftree-vectorize", "-std=gnu99", "-w", "-fPIC", "-pthread", "-D_GNU_SOURCE"]
    lib = os.path.join(bin_dir, "libfflib.so")
    run([cc] + common + inc + ["-shared", "-o", lib] + lib_sources +
        ["-x", "c", "-std=gnu11", os.path.join(SHIM, "mpi_shim.c"), "-lm"])
    run([cc, "-O2", "-o", os.path.join(bin_dir, "shimrun"), os.path.join(SHIM, "shimrun.c")])
    built = []
    for name in PROGRAMS:
        c = os.path.join(src_dst, "evaluation", name + ".c")
        if not os.path.exists(c):
            continue
        run([cc] + common + inc + ["-o", os.path.join(bin_dir, name), c, "-L", bin_dir, "-lfflib",
                                    "-Wl,-rpath,$ORIGIN", "-lm"])
        built.append(name)
    return "built libfflib.so, shimrun and %d programs in %s" % (len(built), bin_dir)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--source", default=DEFAULT_SOURCE)
    ap.add_argument("--force", action="store_true", help="copy the sources again")
    a = ap.parse_args()
    print(build(a.source, a.force))
    sys.exit(0)
