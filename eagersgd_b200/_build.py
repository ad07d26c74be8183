"""In-tree native builds.

Two shared libraries are produced under ``eagersgd_b200/_lib``:

* ``libesgd_host.so``  — C++ control plane and CPU backend (g++), no CUDA needed;
* ``libesgd_cuda.so``  — every CUDA kernel, compiled for sm_100a only (nvcc).

Both export plain ``extern "C"`` launchers taking raw pointers and a stream, so
they are loaded with ``ctypes`` and rebuilt in seconds.  The arch is pinned
(the reference probes the local GPU instead:
deep500/lv0/operators/tools/get_cuda_arch.cpp:8-33).
"""
from __future__ import annotations

import ctypes
import glob
import os
import shutil
import subprocess
import threading

_ROOT = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_ROOT, "csrc")
LIBDIR = os.path.join(_ROOT, "_lib")
HOST_LIB = os.path.join(LIBDIR, "libesgd_host.so")
CUDA_LIB = os.path.join(LIBDIR, "libesgd_cuda.so")

CUDA_ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
_lock = threading.Lock()
_cache: dict = {}


def _newest(paths):
    return max((os.path.getmtime(p) for p in paths), default=0.0)


def _sources(sub, exts):
    out = []
    for ext in exts:
        out += glob.glob(os.path.join(CSRC, sub, "*" + ext))
    # *_main.cpp are stand-alone programs (the sanitizer stress driver), not part of the libraries
    return sorted(f for f in out if not f.endswith("_main.cpp"))


def _headers():
    return glob.glob(os.path.join(CSRC, "**", "*.h"), recursive=True) + glob.glob(
        os.path.join(CSRC, "**", "*.cuh"), recursive=True
    )


def _digest(srcs):
    import hashlib

    h = hashlib.sha256()
    for p in sorted(srcs + _headers()):
        h.update(os.path.relpath(p, CSRC).encode())
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def _stale(lib, srcs):
    """Content-hash staleness: file times do not survive a copy of the tree."""
    if not os.path.exists(lib) or not os.path.exists(lib + ".sha"):
        return True
    return open(lib + ".sha").read().strip() != _digest(srcs)


def _stamp(lib, srcs):
    with open(lib + ".sha", "w") as f:
        f.write(_digest(srcs))


class _FileLock:
    """Serialises builds across the ranks of one node."""

    def __init__(self, path):
        self.path = path

    def __enter__(self):
        import fcntl

        os.makedirs(os.path.dirname(self.path), exist_ok=True)
        self.f = open(self.path, "w")
        fcntl.flock(self.f, fcntl.LOCK_EX)
        return self

    def __exit__(self, *a):
        import fcntl

        fcntl.flock(self.f, fcntl.LOCK_UN)
        self.f.close()


def nvcc_path():
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    return None


def build_host(force: bool = False, verbose: bool = False) -> str:
    srcs = _sources("host", [".cpp"])
    if not force and not _stale(HOST_LIB, srcs):
        return HOST_LIB
    with _FileLock(os.path.join(LIBDIR, ".build.lock")):
        if not force and not _stale(HOST_LIB, srcs):
            return HOST_LIB
        return _build_host_locked(srcs, verbose)


def _build_host_locked(srcs, verbose):
    cmd = ["g++", "-O3", "-std=c++17", "-fPIC", "-shared", "-pthread", "-ftree-vectorize", "-Wall",
           "-I", CSRC, "-o", HOST_LIB + ".tmp"] + srcs + ["-lrt"]
    if verbose:
        print(" ".join(cmd))
    subprocess.run(cmd, check=True)
    os.replace(HOST_LIB + ".tmp", HOST_LIB)
    _stamp(HOST_LIB, srcs)
    return HOST_LIB


def build_cuda(force: bool = False, verbose: bool = False, jobs: int = 8) -> str:
    srcs = _sources("cuda", [".cu"])
    if not force and not _stale(CUDA_LIB, srcs):
        return CUDA_LIB
    with _FileLock(os.path.join(LIBDIR, ".build.lock")):
        if not force and not _stale(CUDA_LIB, srcs):
            return CUDA_LIB
        return _build_cuda_locked(srcs, force, verbose, jobs)


def _build_cuda_locked(srcs, force, verbose, jobs):
    nvcc = nvcc_path()
    if nvcc is None:
        raise RuntimeError("nvcc not found: cannot build the sm_100a kernels")
    os.makedirs(LIBDIR, exist_ok=True)
    objdir = os.path.join(LIBDIR, "obj")
    os.makedirs(objdir, exist_ok=True)
    hdr_time = _newest(_headers())
    procs, objs = [], []
    for src in srcs:
        obj = os.path.join(objdir, os.path.basename(src) + ".o")
        objs.append(obj)
        if not force and os.path.exists(obj) and os.path.getmtime(obj) > max(os.path.getmtime(src), hdr_time):
            if os.path.exists(obj + ".log") and "error" not in open(obj + ".log").read():
                continue
        cmd = [nvcc, "-O3", "-std=c++17", "-lineinfo", "--use_fast_math", "-Xcompiler", "-fPIC",
               "-Xptxas", "-v", "-I", CSRC] + CUDA_ARCH_FLAGS + ["-c", src, "-o", obj]
        if verbose:
            print(" ".join(cmd))
        log = open(obj + ".log", "w")
        procs.append((subprocess.Popen(cmd, stdout=log, stderr=subprocess.STDOUT), src, obj, log))
        while len([p for p in procs if p[0].poll() is None]) >= jobs:
            procs[0][0].wait()
    for proc, src, obj, log in procs:
        rc = proc.wait()
        log.close()
        if rc != 0:
            raise RuntimeError("nvcc failed for %s:\n%s" % (src, open(obj + ".log").read()[-4000:]))
    cmd = [nvcc, "-shared", "-o", CUDA_LIB + ".tmp"] + objs + CUDA_ARCH_FLAGS
    subprocess.run(cmd, check=True)
    os.replace(CUDA_LIB + ".tmp", CUDA_LIB)
    _stamp(CUDA_LIB, srcs)
    return CUDA_LIB


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_host(force, verbose)
    build_cuda(force, verbose)


def load_host() -> ctypes.CDLL:
    with _lock:
        if "host" not in _cache:
            _cache["host"] = ctypes.CDLL(build_host())
        return _cache["host"]


def load_cuda() -> ctypes.CDLL:
    """Load the CUDA kernel library.  Fails loudly: there is no fallback path."""
    with _lock:
        if "cuda" not in _cache:
            if os.path.exists(CUDA_LIB) and nvcc_path() is None:
                path = CUDA_LIB  # GPU box without a compiler: use the shipped build
            else:
                path = build_cuda()
            _cache["cuda"] = ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)
        return _cache["cuda"]


def write_pkgconfig() -> str:
    """Write ``_lib/pkgconfig/esgd_host.pc`` so that C and C++ programs can compile and link against the host
    library (operation runtime ``host/oprt.h``, CPU channel) with ``pkg-config --cflags --libs esgd_host`` —
    what the reference's ``fflib.pc`` does for ``libfflib.so`` (fflib2 CMakeLists.txt:83-96, fflib.pc.in)."""
    d = os.path.join(LIBDIR, "pkgconfig")
    os.makedirs(d, exist_ok=True)
    path = os.path.join(d, "esgd_host.pc")
    with open(path, "w") as f:
        f.write("prefix=%s\nlibdir=%s\nincludedir=%s\n\nName: esgd_host\nDescription: eager-SGD host runtime "
                "(persistent dependency-triggered operations, schedules, CPU partial allreduce)\nVersion: 0.2.0\n"
                "Libs: -L${libdir} -lesgd_host -Wl,-rpath,${libdir} -pthread\nCflags: -I${includedir}\n"
                % (os.path.dirname(LIBDIR), LIBDIR, CSRC))
    return path


def main(argv=None) -> int:
    import sys
    argv = sys.argv[1:] if argv is None else argv
    build_all(force="--force" in argv, verbose=True)
    print("built", HOST_LIB, CUDA_LIB)
    print("pkg-config file:", write_pkgconfig())
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
