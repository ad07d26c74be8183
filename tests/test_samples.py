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
])
def test_sample_runs(script, args):
    r = subprocess.run([sys.executable, os.path.join(ROOT, "samples", script)] + args, capture_output=True, text=True,
                       timeout=600, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
