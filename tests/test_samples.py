"""The example programs run and check themselves (CPU ones here)."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("script,args", [
    ("train_mnist.py", ["--epochs", "1", "--train-size", "512"]),
    ("custom_operator.py", []),
    ("op_runtime_schedule.py", ["--ranks", "3"]),
    ("partial_allreduce_cpu.py", ["--mode", "solo", "--steps", "8"]),
    ("partial_allreduce_cpu.py", ["--mode", "majority", "--steps", "8"]),
    ("graph_inference.py", []),
    ("lstm_video_classifier.py", ["--steps", "2", "--hidden", "32", "--max-length", "20", "--batch", "4"]),
    ("ucf101_resnetlstm.py", ["--resnet-size", "8", "--hidden", "16", "--max-steps", "2", "--skip-frames", "4"]),
    ("train_until.py", ["80", "--max-epochs", "3", "--train-size", "512"]),
    ("accelegrad.py", ["--epochs", "1", "--train-size", "512"]),
    ("dataset_latency.py", ["--batches", "2"]),
    ("mnist_bias.py", []),
    ("network_inference.py", []),
    ("network_inference.py", ["reference"]),
    ("onnxtest.py", ["all"]),
    ("synthetic_dataset.py", ["--resnet-size", "8", "--size", "32", "--batch", "8", "--steps", "2"]),
    ("imbalance_modes_cpu.py", ["--ranks", "3", "--steps", "15", "--buckets", "2"]),
    ("deepbench/gemm_overhead.py", ["--limit", "2", "--reruns", "2"]),
    ("deepbench/conv_overhead.py", ["--limit", "1", "--reruns", "2"]),
])
def test_sample_runs(script, args):
    r = subprocess.run([sys.executable, os.path.join(ROOT, "samples", script)] + args, capture_output=True, text=True,
                       timeout=600, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]


@pytest.mark.gpu
def test_peer_collectives_sample_runs_emulated_on_one_gpu():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "samples", "peer_collectives.py"), "--emulate", "4"],
                       capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "expected 6.0" in r.stdout and "[6.0, 6.0]" in r.stdout and "status words: [0, 0, 0, 0]" in r.stdout


@pytest.mark.parametrize("scheme", ["solo", "pssgd", "mavg"])
def test_distributed_training_sample_on_cpu_ranks(scheme):
    """samples/distributed_training.py as two gloo ranks: an eager scheme, a parameter server and model averaging."""
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(ROOT, "samples", "distributed_training.py"), "--scheme", scheme,
           "--steps", "12", "--dim", "64", "--sleep-ms", "2"]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="1")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env, cwd=ROOT)
    assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
