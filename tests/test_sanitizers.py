"""Race and memory checks of the host control plane: the protocol source shared with the CUDA kernels and the
operation runtime run under ThreadSanitizer and AddressSanitizer + UBSan through a C++ stress driver."""
import os
import shutil
import subprocess

import pytest

HOST = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "eagersgd_b200", "csrc", "host")


@pytest.mark.parametrize("flags,needle", [("-fsanitize=thread", "ThreadSanitizer"),
                                          ("-fsanitize=address,undefined", "Sanitizer")])
def test_stress_driver_is_clean(tmp_path, flags, needle):
    if shutil.which("g++") is None:
        pytest.skip("no host compiler")
    exe = str(tmp_path / "stress")
    build = subprocess.run(["g++", "-std=c++17", "-O1", "-g", flags, "-Wno-tsan", "stress_main.cpp", "cpu_channel.cpp",
                            "oprt.cpp", "-lpthread", "-o", exe], cwd=HOST, capture_output=True, text=True)
    if build.returncode != 0 and "sanitize" in build.stderr and "cannot find" in build.stderr:
        pytest.skip("sanitizer runtime not installed")
    assert build.returncode == 0, build.stderr[-3000:]
    run = subprocess.run([exe, "4", "300"], capture_output=True, text=True, timeout=600)
    out = run.stdout + run.stderr
    assert run.returncode == 0, out[-3000:]
    assert needle not in out, out[-3000:]
    assert out.count("on every rank") == 7 and "runtime allreduce: 4 ranks" in out
    assert "runtime schedule cycles: 4 ranks ok" in out
    assert "runtime partial allreduce: 4 ranks x 6 cycles x 16 posts of 8 elements ok" in out
    assert "runtime partial allreduce: 4 ranks x 2 cycles x 8 posts of 8192 elements ok" in out
