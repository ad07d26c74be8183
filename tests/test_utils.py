import pytest
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_fork_relaunches_script_as_ranks(tmp_path):
    script = tmp_path / "prog.py"
    script.write_text(textwrap.dedent('''
        import os, sys
        sys.path.insert(0, %r)
        from eagersgd_b200.utils import fork, rank_env
        role = fork(2, timeout=300)
        if role == "child":
            import torch.distributed as dist, torch
            dist.init_process_group("gloo")
            t = torch.tensor([float(rank_env()["rank"] + 1)])
            dist.all_reduce(t)
            open(os.path.join(%r, "rank%%d.txt" %% rank_env()["rank"]), "w").write(str(t.item()))
            dist.destroy_process_group()
        else:
            print("parent done")
    ''' % (ROOT, str(tmp_path))))
    r = subprocess.run([sys.executable, str(script)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-1500:]
    assert "parent done" in r.stdout
    assert (tmp_path / "rank0.txt").read_text() == "3.0" and (tmp_path / "rank1.txt").read_text() == "3.0"


def test_device_descriptors_and_peaks(tmp_path):
    import json
    from eagersgd_b200.utils import CPUDevice, GPUDevice, describe, measured_peaks
    assert not CPUDevice().is_gpu() and GPUDevice(1).is_gpu() and repr(GPUDevice(1)) == "cuda:1"
    assert str(CPUDevice().torch_device()) == "cpu"
    p = tmp_path / "peaks.json"
    p.write_text(json.dumps({"hbm_gbs": 6000.0, "bf16_tflops": 1500.0}))
    assert measured_peaks(str(p))["source"] == "measured" and measured_peaks(str(tmp_path / "none.json"))["source"] == "fallback"
    d = describe()
    assert d["nominal"]["sms"] == 148 and d["peaks"]["hbm_gbs"] > 0


def test_zero_arena_hands_out_aligned_slices_and_falls_back():
    import torch
    from eagersgd_b200.ops import functional as ops
    a = ops.zeros_f32((3, 5), torch.device("cpu"))            # inactive: plain zeros
    assert a.shape == (3, 5) and float(a.abs().sum()) == 0.0
    with ops.zero_arena("cpu", 256):
        b = ops.zeros_f32((2, 10), torch.device("cpu"))
        c = ops.zeros_f32((7,), torch.device("cpu"))
        assert b.data_ptr() % 256 == c.data_ptr() % 256       # 64-float granularity
        assert c.data_ptr() - b.data_ptr() == 64 * 4
        b.add_(1.0)
        big = ops.zeros_f32((1000,), torch.device("cpu"))     # does not fit: falls back
        assert float(big.sum()) == 0.0 and big.numel() == 1000
    with ops.zero_arena("cpu", 256):                           # a new step starts from zeros again
        b2 = ops.zeros_f32((2, 10), torch.device("cpu"))
        assert float(b2.sum()) == 0.0
    assert float(ops.zeros_f32((4,), torch.device("cpu")).sum()) == 0.0
    # the cleared prefix follows the largest use so far, whatever the order of small and large steps
    for sizes in ([10], [10, 70, 5], [3], [10, 70, 5]):
        with ops.zero_arena("cpu", 256):
            got = [ops.zeros_f32((k,), torch.device("cpu")) for k in sizes]
            assert all(float(t.abs().sum()) == 0.0 for t in got), sizes
            for t in got:
                t.fill_(7.0)


def test_host_library_links_from_c_through_pkgconfig(tmp_path):
    """A C program includes host/oprt.h, links libesgd_host through the generated pkg-config file and runs a
    two-rank allreduce of the operation runtime."""
    import os
    import shutil
    import subprocess
    from eagersgd_b200 import _build
    if shutil.which("gcc") is None:
        pytest.skip("no C compiler")
    _build.build_host()
    pc = _build.write_pkgconfig()
    text = open(pc).read()
    flags = {}
    for line in text.splitlines():
        if "=" in line and ":" not in line.split("=")[0]:
            k, v = line.split("=", 1)
            flags[k] = v
    expand = lambda s: s.replace("${libdir}", flags["libdir"]).replace("${includedir}", flags["includedir"])
    cflags = expand([l for l in text.splitlines() if l.startswith("Cflags:")][0].split(":", 1)[1]).split()
    libs = expand([l for l in text.splitlines() if l.startswith("Libs:")][0].split(":", 1)[1]).split()
    src = tmp_path / "prog.c"
    src.write_text("""
#include <stdio.h>
#include <pthread.h>
#include "host/oprt.h"
static rt_world* w;
static int ok[2];
static void* body(void* arg) {
  int r = (int)(long)arg;
  rt_rank* c = rt_world_rank(w, r);
  int snd[4] = {r + 1, 2, 3, 4}, rcv[4] = {0, 0, 0, 0};
  rt_buf bs = rt_buffer_create(c, snd, 4, RT_INT32), br = rt_buffer_create(c, rcv, 4, RT_INT32);
  rt_sched s = rt_allreduce(c, bs, br, 1, RT_SUM);
  rt_schedule_post(c, s);
  ok[r] = rt_schedule_wait(c, s, 10.0) == RT_SUCCESS && rcv[0] == 3 && rcv[3] == 8;
  rt_schedule_delete(c, s);
  return 0;
}
int main(void) {
  pthread_t t[2];
  w = rt_world_create(2);
  for (long r = 0; r < 2; ++r) pthread_create(&t[r], 0, body, (void*)r);
  for (int r = 0; r < 2; ++r) pthread_join(t[r], 0);
  rt_world_destroy(w);
  printf(ok[0] && ok[1] ? "PASSED\\n" : "FAILED\\n");
  return !(ok[0] && ok[1]);
}
""")
    exe = str(tmp_path / "prog")
    subprocess.run(["gcc", "-O1", str(src), "-o", exe] + cflags + libs, check=True)
    out = subprocess.run([exe], capture_output=True, text=True, timeout=60)
    assert out.returncode == 0 and "PASSED" in out.stdout, out.stdout + out.stderr


def test_nvtx_ranges_are_free_when_off(monkeypatch):
    """``nvtx_range`` hands out one shared no-op context unless ESGD_NVTX=1."""
    import eagersgd_b200.utils.nvtx as nv
    monkeypatch.setattr(nv, "_ON", None)
    monkeypatch.setenv("ESGD_NVTX", "0")
    a, b = nv.nvtx_range("x"), nv.nvtx_range("y")
    assert a is b and not nv.nvtx_enabled()
    with a:
        pass
    monkeypatch.setattr(nv, "_ON", None)
    monkeypatch.setenv("ESGD_NVTX", "1")
    assert nv.nvtx_enabled() and nv.nvtx_range("x") is not a
    monkeypatch.setattr(nv, "_ON", None)


def test_collective_plans_pair_every_sender_with_a_reader():
    """The masks of the peer-memory collectives, for every rank of worlds of 2 to 8: whoever a rank publishes to
    reads from it and vice versa (an unmatched side would wait until its time limit on a GPU)."""
    from eagersgd_b200.parallel.peer_collectives import _Plan
    for world in range(2, 9):
        plans = [_Plan(r, world) for r in range(world)]
        for name, args in (("bcast", (0,)), ("bcast", (world - 1,)), ("gather", (1 % world,)), ("allgather", ()),
                           ("neighbours", ())):
            masks = [getattr(p, name)(*args) for p in plans]
            for a in range(world):
                dst_a, src_a, slot_a = masks[a]
                assert not dst_a >> a & 1 and not src_a >> a & 1            # nobody sends to itself
                for b in range(world):
                    if a != b:
                        assert bool(dst_a >> b & 1) == bool(masks[b][1] >> a & 1), (name, world, a, b)
        root = 1 % world
        assert [p.gather(root)[2] for p in plans] == [r if r == root else -1 for r in range(world)]
        assert all(p.allgather()[2] == r for r, p in enumerate(plans))


def test_bench_clock_sampler_parses_a_fake_nvidia_smi(tmp_path, monkeypatch):
    """The bench's clock record: median SM clock, maximum, and the throttle reasons seen during the timed region,
    from the lines ``nvidia-smi -lms`` prints (here a stand-in script, so that the parsing is tested without a GPU)."""
    import importlib.util
    import os
    import stat
    import time
    fake = tmp_path / "nvidia-smi"
    fake.write_text("#!/bin/bash\n"
                    "echo '1965, 1965, 400.1, Not Active, Not Active, Not Active, Not Active'\n"
                    "echo '1410, 1965, 998.0, Not Active, Not Active, Not Active, Active'\n"
                    "echo '1400, 1965, 999.5, Not Active, Not Active, Not Active, Active'\n"
                    "echo 'garbage line'\n"
                    "sleep 5\n")
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("PATH", str(tmp_path) + os.pathsep + os.environ["PATH"])
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(root, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    s = bench.ClockSampler(0)
    s.start()
    time.sleep(0.5)
    rec = s.stop()
    assert rec == {"sm_mhz": 1410.0, "sm_max_mhz": 1965.0, "samples": 3, "reasons": ["sw_power_cap"]}
    monkeypatch.setenv("PATH", str(tmp_path / "nothing"))
    s = bench.ClockSampler(0)
    s.start()
    assert s.stop()["reasons"] == ["nvidia-smi unavailable"]


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_c_sample_of_the_partial_allreduce(tmp_path, mode):
    """samples/c/solo_allreduce.c — the reference's rsgd.c loop written against host/esgd_channel.h — compiles with
    the flags of the pkg-config file and passes its own checks in solo, majority and synchronous mode."""
    import os
    import shutil
    import subprocess
    from eagersgd_b200 import _build
    if shutil.which("gcc") is None:
        pytest.skip("no C compiler")
    _build.build_host()
    text = open(_build.write_pkgconfig()).read()
    var = dict(l.split("=", 1) for l in text.splitlines() if "=" in l and ":" not in l.split("=")[0])
    expand = lambda s: s.replace("${libdir}", var["libdir"]).replace("${includedir}", var["includedir"])
    cflags = expand([l for l in text.splitlines() if l.startswith("Cflags:")][0].split(":", 1)[1]).split()
    libs = expand([l for l in text.splitlines() if l.startswith("Libs:")][0].split(":", 1)[1]).split()
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe = str(tmp_path / "solo_allreduce")
    subprocess.run(["gcc", "-O2", "-Wall", "-Werror", os.path.join(root, "samples", "c", "solo_allreduce.c")] + cflags + libs +
                   ["-o", exe], check=True, capture_output=True, text=True)
    r = subprocess.run([exe, "3", "2048", "6", str(mode)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "PASSED" in r.stdout and "replicas agree" in r.stdout, r.stdout + r.stderr


@pytest.mark.parametrize("mode", [0, 1])
def test_c_sample_of_the_runtime_partial_allreduce(tmp_path, mode):
    """samples/c/rt_partial_allreduce.c — the reference's rsgd.c / randomsgd.c loop on the operation runtime's solo and
    majority allreduce schedules, from plain C — builds with the pkg-config flags and passes its own conservation check."""
    import os
    import shutil
    import subprocess
    from eagersgd_b200 import _build
    if shutil.which("gcc") is None:
        pytest.skip("no C compiler")
    _build.build_host()
    text = open(_build.write_pkgconfig()).read()
    var = dict(l.split("=", 1) for l in text.splitlines() if "=" in l and ":" not in l.split("=")[0])
    expand = lambda s: s.replace("${libdir}", var["libdir"]).replace("${includedir}", var["includedir"])
    cflags = expand([l for l in text.splitlines() if l.startswith("Cflags:")][0].split(":", 1)[1]).split()
    libs = expand([l for l in text.splitlines() if l.startswith("Libs:")][0].split(":", 1)[1]).split()
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe = str(tmp_path / "rt_partial_allreduce")
    subprocess.run(["gcc", "-O2", "-Wall", "-Werror", os.path.join(root, "samples", "c", "rt_partial_allreduce.c")] + cflags +
                   libs + ["-lpthread", "-o", exe], check=True, capture_output=True, text=True)
    r = subprocess.run([exe, "4", "4096", "12", str(mode), "5"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "PASSED" in r.stdout and "2 synchronous" in r.stdout, r.stdout + r.stderr


def test_end_barrier_is_a_no_op_outside_a_process_group():
    from eagersgd_b200.utils.launch import end_barrier, rank_env
    end_barrier()                                               # no group: returns at once
    assert rank_env()["world"] >= 1


def test_every_name_the_migration_guide_gives_can_be_imported():
    """docs/migrating.md maps the reference's names to this package's: each dotted ``eagersgd_b200...`` name in it exists,
    and so does every ``rt_`` function it names in the C header."""
    import importlib
    import os
    import re
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    text = open(os.path.join(root, "docs", "migrating.md")).read()
    names = sorted(set(re.findall(r"`(eagersgd_b200(?:\.[A-Za-z_][A-Za-z_0-9]*)+)", text)))
    assert len(names) > 25
    for n in names:
        parts = n.split(".")
        for k in range(len(parts), 0, -1):
            try:
                obj = importlib.import_module(".".join(parts[:k]))
                break
            except ImportError:
                continue
        for a in parts[k:]:
            assert hasattr(obj, a), n
            obj = getattr(obj, a)
    header = open(os.path.join(root, "eagersgd_b200", "csrc", "host", "oprt.h")).read()
    for fn in sorted(set(re.findall(r"`(rt_[a-z_]+)", text))):
        if fn.endswith("_"):
            assert fn in header, fn                              # a prefix such as rt_schedule_
        else:
            assert re.search(r"\b%s\w*\(" % fn, header), fn


def test_the_readme_snippet_names_resolve():
    """``import eagersgd_b200 as es`` alone gives access to the sub-packages the README uses."""
    import subprocess
    import sys
    code = ("import eagersgd_b200 as es\n"
            "assert callable(es.train.prepare_model) and callable(es.data.ShuffleSampler) and callable(es.models.create_model)\n"
            "assert callable(es.SoloAllreduceOptimizer) and callable(es.PartialAllreduce) and callable(es.init)\n"
            "assert callable(es.graph.load_onnx) and callable(es.ckpt.save) and callable(es.recipes.run_recipe)\n"
            "try:\n    es.no_such_thing\nexcept AttributeError:\n    print('ok')\n")
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=root, timeout=300)
    assert r.returncode == 0 and r.stdout.strip() == "ok", r.stderr[-2000:]
