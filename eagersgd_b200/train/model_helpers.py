"""Small helpers a training main calls, and the helpers its tests use.

``past_stop_threshold``, ``generate_synthetic_data`` and ``apply_clean`` stand where the reference's run loop uses
official/utils/misc/model_helpers.py:29-93; ``MockBenchmarkLogger`` and ``run_synthetic`` where its tests use
official/utils/testing/mock_lib.py:23-36 and integration.py:32-65 (a minimal run of a main on synthetic data, to
find errors along the whole code path).
"""
from __future__ import annotations

import numbers
import os
import shutil
import tempfile
from typing import Callable, Optional, Sequence

import torch


def past_stop_threshold(stop_threshold, eval_metric) -> bool:
    """Whether training should stop: the metric has reached the threshold.  No threshold: never."""
    if stop_threshold is None:
        return False
    if not isinstance(stop_threshold, numbers.Number):
        raise ValueError("the stop threshold must be a number")
    if not isinstance(eval_metric, numbers.Number):
        raise ValueError("the metric checked against the stop threshold must be a number")
    return eval_metric >= stop_threshold


def per_device_batch_size(batch_size: int, num_gpus: int) -> int:
    """The batch of one GPU when ``batch_size`` is the global one: it has to divide evenly
    (official/utils/misc/distribution_utils.py:50-79)."""
    if num_gpus <= 1:
        return batch_size
    if batch_size % num_gpus:
        raise ValueError("When running with multiple GPUs, batch size must be a multiple of the number of available GPUs. "
                         "Found %d GPUs with a batch size of %d; try --batch_size=%d instead."
                         % (num_gpus, batch_size, batch_size - batch_size % num_gpus))
    return batch_size // num_gpus


def generate_synthetic_data(input_shape: Sequence[int], input_value=0, input_dtype=torch.float32,
                            label_shape: Optional[Sequence[int]] = None, label_value=0, label_dtype=torch.int64,
                            batches: Optional[int] = None):
    """An endless (or ``batches`` long) iterator of constant batches: ``x`` alone, or ``(x, y)`` when
    ``label_shape`` is given.  The tensors are made once and handed out again and again."""
    x = torch.full(tuple(input_shape), input_value, dtype=input_dtype)
    y = torch.full(tuple(label_shape), label_value, dtype=label_dtype) if label_shape is not None else None
    k = 0
    while batches is None or k < batches:
        yield (x, y) if y is not None else x
        k += 1


def apply_clean(clean: bool, model_dir: str) -> None:
    """``--clean``: start from an empty model directory."""
    if clean and model_dir and os.path.isdir(model_dir):
        shutil.rmtree(model_dir)


class MockBenchmarkLogger:
    """A logger that only remembers what it was given (for tests of code that logs metrics)."""

    def __init__(self):
        self.logged_metric, self.logged_run_info, self.logged_evaluation = [], [], []

    def log_metric(self, name, value, unit=None, global_step=None, extras=None):
        self.logged_metric.append({"name": name, "value": float(value), "unit": unit, "global_step": global_step,
                                   "extras": extras})

    def log_evaluation_result(self, eval_results):
        self.logged_evaluation.append(dict(eval_results))
        for k, v in eval_results.items():
            if k != "global_step" and isinstance(v, numbers.Number):
                self.log_metric(k, v, global_step=eval_results.get("global_step"))

    def log_run_info(self, *args, **kwargs):
        self.logged_run_info.append((args, kwargs))

    def on_finish(self, status):
        self.status = status


def run_synthetic(main: Callable[[Sequence[str]], int], tmp_root: str, extra_flags: Optional[Sequence[str]] = None,
                  synth: bool = True, max_train: Optional[int] = 1) -> int:
    """A minimal run of a training main (``main(argv) -> exit code``) in a scratch model directory that is removed
    afterwards: one epoch, one evaluation, synthetic data, at most ``max_train`` steps."""
    model_dir = tempfile.mkdtemp(dir=tmp_root)
    args = ["--model_dir", model_dir, "--train_epochs", "1", "--epochs_between_evals", "1"] + list(extra_flags or [])
    if synth:
        args.append("--use_synthetic_data")
    if max_train is not None:
        args += ["--max_train_steps", str(max_train)]
    try:
        return main(args)
    finally:
        shutil.rmtree(model_dir, ignore_errors=True)
