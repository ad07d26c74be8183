"""Benchmark loggers and throughput hooks.

``BaseBenchmarkLogger`` (stdout) and ``BenchmarkFileLogger`` (``metric.log`` JSON lines plus
``benchmark_run.log`` with run and machine information) follow official/utils/logs/logger.py:
57-218; ``ExamplesPerSecondHook`` follows official/utils/logs/hooks.py:28-127 (average and
current examples/s every N steps); ``LoggingMetricHook`` follows metric_hook.py:24-97; the
training log line is the reference's formatter (resnet_run_loop_solo_imagenet_300.py:582-623).
Only rank 0 logs.
"""
from __future__ import annotations

import contextlib
import datetime
import json
import os
import platform
import threading
import time
from typing import Dict, Optional

import torch

RUN_STATUS_SUCCESS, RUN_STATUS_FAILURE, RUN_STATUS_RUNNING = "success", "failure", "running"


class BaseBenchmarkLogger:
    def log_evaluation_result(self, eval_results: Dict):
        step = eval_results.get("global_step", 0)
        for k, v in sorted(eval_results.items()):
            if k != "global_step":
                self.log_metric(k, v, global_step=step)

    def log_metric(self, name, value, unit=None, global_step=None, extras=None):
        print("Benchmark metric:", _metric(name, value, unit, global_step, extras))

    def log_run_info(self, model_name, dataset_name, run_params, test_id=None):
        print("Benchmark run:", gather_run_info(model_name, dataset_name, run_params, test_id))

    def on_finish(self, status):
        pass


class BenchmarkFileLogger(BaseBenchmarkLogger):
    def __init__(self, logging_dir: str):
        self.dir = logging_dir
        os.makedirs(logging_dir, exist_ok=True)
        self._f = open(os.path.join(logging_dir, "metric.log"), "a")

    def log_metric(self, name, value, unit=None, global_step=None, extras=None):
        self._f.write(json.dumps(_metric(name, value, unit, global_step, extras)) + "\n")
        self._f.flush()

    def log_run_info(self, model_name, dataset_name, run_params, test_id=None):
        with open(os.path.join(self.dir, "benchmark_run.log"), "w") as f:
            json.dump(gather_run_info(model_name, dataset_name, run_params, test_id), f)
            f.write("\n")

    def on_finish(self, status):
        """Close the metric file and leave the run's final status beside it (the reference keeps the status in
        its BigQuery run-status table, logger.py:293-300; with no such service here it is a one-line file)."""
        self.status = status
        if not self._f.closed:
            self._f.flush()
            self._f.close()
        with open(os.path.join(self.dir, "run_status.log"), "w") as f:
            json.dump({"run_status": status}, f)
            f.write("\n")


_benchmark_logger: Optional[BaseBenchmarkLogger] = None
_logger_lock = threading.Lock()


def config_benchmark_logger(flag_obj=None) -> BaseBenchmarkLogger:
    """Set the process-wide benchmark logger from a flags object (``benchmark_logger_type``, ``benchmark_log_dir``);
    without one, or with the base type, metrics go to standard output (logger.py:56-86).  The reference's third type
    uploads to BigQuery; with no network here a request for it is an error like any unknown type."""
    global _benchmark_logger
    with _logger_lock:
        kind = getattr(flag_obj, "benchmark_logger_type", None) or "BaseBenchmarkLogger"
        if kind == "BaseBenchmarkLogger":
            _benchmark_logger = BaseBenchmarkLogger()
        elif kind == "BenchmarkFileLogger":
            _benchmark_logger = BenchmarkFileLogger(flag_obj.benchmark_log_dir)
        else:
            raise ValueError("Unrecognized benchmark_logger_type: %s" % kind)
        return _benchmark_logger


def get_benchmark_logger() -> BaseBenchmarkLogger:
    """The process-wide logger (a standard-output one if nothing was configured)."""
    if _benchmark_logger is None:
        config_benchmark_logger()
    return _benchmark_logger


def _metric(name, value, unit, global_step, extras):
    return {"name": name, "value": float(value), "unit": unit, "global_step": global_step,
            "timestamp": datetime.datetime.now(datetime.timezone.utc).strftime("%Y-%m-%dT%H:%M:%S.%fZ"),
            "extras": [{"name": k, "value": str(v)} for k, v in sorted((extras or {}).items())]}


def gather_run_info(model_name, dataset_name, run_params, test_id=None) -> dict:
    info = {"model_name": model_name, "dataset": {"name": dataset_name}, "machine_config": {},
            "test_id": test_id, "run_date": datetime.datetime.now(datetime.timezone.utc).strftime("%Y-%m-%dT%H:%M:%S.%fZ"),
            "torch_version": torch.__version__,
            "run_parameters": [{"name": k, "value": str(v)} for k, v in sorted((run_params or {}).items())]}
    info["machine_config"]["cpu_info"] = {"num_cores": os.cpu_count(), "cpu_info": platform.processor()}
    if torch.cuda.is_available():
        info["machine_config"]["gpu_info"] = {"count": torch.cuda.device_count(),
                                              "model": torch.cuda.get_device_name(0)}
    try:                                      # memory of the host, when psutil is there (logger.py:407-416)
        import psutil
        vm = psutil.virtual_memory()
        info["machine_config"]["memory_total"], info["machine_config"]["memory_available"] = vm.total, vm.available
    except ImportError:
        pass
    # the switches of this framework and of its libraries that were set for the run (logger.py:361-366 lists TF_*)
    info["environment_variables"] = [{"name": k, "value": v} for k, v in sorted(os.environ.items())
                                     if k.startswith(("ESGD_", "NCCL_", "CUDA_", "OMP_"))]
    return info


@contextlib.contextmanager
def benchmark_context(logger: BaseBenchmarkLogger):
    """Reports success or failure of the run to the logger (logger.py:96-106)."""
    try:
        yield
        logger.on_finish(RUN_STATUS_SUCCESS)
    except Exception:
        logger.on_finish(RUN_STATUS_FAILURE)
        raise


class ExamplesPerSecondHook:
    """Call ``after_step()`` once per training step."""

    def __init__(self, batch_size: int, every_n_steps: int = 100, warm_steps: int = 0,
                 metric_logger: Optional[BaseBenchmarkLogger] = None):
        self.batch_size, self.every, self.warm = batch_size, every_n_steps, warm_steps
        self.logger = metric_logger or BaseBenchmarkLogger()
        self.step, self.total_time, self.total_steps, self._t = 0, 0.0, 0, None

    def after_step(self):
        now = time.time()
        self.step += 1
        if self._t is None or self.step <= self.warm:
            self._t = now
            return None
        if (self.step - self.warm) % self.every == 0:
            elapsed = now - self._t
            self._t = now
            self.total_time += elapsed
            self.total_steps += self.every
            avg = self.batch_size * self.total_steps / self.total_time
            cur = self.batch_size * self.every / elapsed
            self.logger.log_metric("average_examples_per_sec", avg, global_step=self.step)
            self.logger.log_metric("current_examples_per_sec", cur, global_step=self.step)
            return avg, cur
        return None


class ProfilerHook:
    """Every ``save_steps`` steps, profile one training step and write a Chrome trace
    (``timeline-<step>.json``) into ``output_dir`` — the reference's ProfilerHook
    (official/utils/logs/hooks_helper.py:98-110: tf.train.ProfilerHook(save_steps=1000)).
    Use ``with hook.step(global_step):`` around the training step."""

    def __init__(self, output_dir: str, save_steps: int = 1000, first_step: int = 10):
        self.dir, self.every, self.first = output_dir, max(int(save_steps), 1), first_step
        self.written = []

    def step(self, global_step: int):
        import contextlib
        if global_step != self.first and (global_step == 0 or global_step % self.every != 0):
            return contextlib.nullcontext()
        return self._profiled(global_step)

    def _profiled(self, global_step: int):
        import contextlib
        import os
        import torch

        @contextlib.contextmanager
        def ctx():
            acts = [torch.profiler.ProfilerActivity.CPU]
            if torch.cuda.is_available():
                acts.append(torch.profiler.ProfilerActivity.CUDA)
            with torch.profiler.profile(activities=acts) as prof:
                yield
                if torch.cuda.is_available():
                    torch.cuda.synchronize()
            os.makedirs(self.dir, exist_ok=True)
            path = os.path.join(self.dir, "timeline-%d.json" % global_step)
            prof.export_chrome_trace(path)
            self.written.append(path)
        return ctx()


HOOKS = ("LoggingTensorHook", "ExamplesPerSecondHook", "ProfilerHook", "LoggingMetricHook")


def parse_hooks(spec: str):
    """``--hooks`` value -> the set of hook names (case-insensitive, as hooks_helper.get_train_hooks accepts)."""
    by_lower = {h.lower(): h for h in HOOKS}
    out = set()
    for name in (spec or "").split(","):
        name = name.strip().lower()
        if not name:
            continue
        if name not in by_lower:
            raise ValueError("unknown hook %r: choose from %s" % (name, ", ".join(HOOKS)))
        out.add(by_lower[name])
    return out


class LoggingMetricHook:
    def __init__(self, metric_logger: BaseBenchmarkLogger, every_n_iter: int = 10):
        self.logger, self.every, self.step = metric_logger, every_n_iter, 0

    def after_step(self, tensors: Dict[str, float]):
        self.step += 1
        if self.step % self.every == 0:
            for k, v in tensors.items():
                self.logger.log_metric(k, v, global_step=self.step)


def training_log_line(epoch: int, step: int, steps_per_epoch: int, lr: float, loss: float, top1: float,
                      top5: float) -> str:
    return ("TRAINING - Epoch: [%d][%d/%d]  LR %.5f  Loss %.4f  Prec@1 %.3f  Prec@5 %.3f"
            % (epoch, step % max(steps_per_epoch, 1), steps_per_epoch, lr, loss, top1, top5))
