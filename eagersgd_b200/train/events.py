"""Training events: hooks the trainer, optimizers, samplers and executors call.

Counterparts of the reference's event classes (deep500/lv2/event.py,
deep500/lv2/events/*.py, deep500/lv1/event.py, deep500/lv2/summaries.py):
TerminalBarEvent, SummaryGeneratorEvent, AccuracyAbortEvent, TimeAbort*Event,
EpochHPSchedule / StepHPSchedule, CsvWriterEvent, LossPlot / BoxPlot generators,
SaveWrongsEvent, plus EpochSummary / TrainingStatistics.  matplotlib is not
available here, so the plot generators write the series they would have drawn as
JSON next to the requested file name.
"""
from __future__ import annotations

import csv
import json
import os
import sys
import time
from typing import Callable, List, Optional


class StopTraining(Exception):
    """Raised by an event to end the run loop cleanly."""


class TrainingEvent:
    """Base class: every hook is optional."""

    def before_training(self, runner, training_stats): ...
    def after_training(self, runner, training_stats): ...
    def before_epoch(self, epoch, runner, training_stats): ...
    def after_epoch(self, epoch, runner, training_stats): ...
    def before_training_step(self, executor, optimizer, inputs): ...
    def after_training_step(self, executor, optimizer, outputs, loss): ...
    def before_training_set(self, runner, training_stats, sampler): ...      # around the training pass of an epoch
    def after_training_set(self, runner, training_stats): ...
    def before_test_batch(self, runner, training_stats, batch): ...           # the reference's names for the test steps
    def after_test_batch(self, runner, training_stats, outputs): ...
    def on_sampler_reset(self, sampler): ...
    def before_test_set(self, runner, training_stats, sampler): ...
    def after_test_set(self, runner, training_stats, sampler): ...
    def before_test_step(self, executor, inputs): ...
    def after_test_step(self, executor, outputs): ...
    def before_optimizer_step(self, executor, optimizer, inputs): ...
    def after_optimizer_step(self, executor, optimizer, loss): ...
    # executor-level (deep500/lv1/event.py)
    def before_executor(self, inputs): ...
    def after_inference(self, outputs): ...
    def after_backprop(self, grads): ...
    # sampler-level
    def before_sampling(self, sampler, batch_size): ...
    def after_sampling(self, sampler, batch_size): ...


class EpochSummary:
    def __init__(self, epoch: int, training: bool):
        self.epoch, self.training = epoch, training
        self.losses: List[float] = []
        self.accuracy: Optional[float] = None
        self.wrong_batches: List = []
        self.time = 0.0
        self.lr: Optional[float] = None
        self.time_used_inference: List[float] = []     # filled by SummaryGeneratorInferenceEvent
        self.time_used_optimizing: List[float] = []

    @property
    def mean_loss(self):
        return sum(self.losses) / max(len(self.losses), 1)

    def to_dict(self) -> dict:
        """One row of the statistics table, with the reference's column names (deep500/lv2/summaries.py:28-39)."""
        inf = self.time_used_inference
        return {"epoch": self.epoch, "avg_loss": self.mean_loss, "accuracy": self.accuracy, "n_batches": len(self.losses),
                "avg_time_inference": sum(inf) / len(inf) if inf else 0.0, "train": self.training, "time_used": self.time,
                "lr": self.lr}


class TrainingStatistics:
    def __init__(self):
        self.train_summaries: List[EpochSummary] = []
        self.test_summaries: List[EpochSummary] = []
        self.start_time = time.time()

    def current_summary(self, training=True) -> EpochSummary:
        return (self.train_summaries if training else self.test_summaries)[-1]

    def clear(self) -> None:
        self.train_summaries, self.test_summaries = [], []
        self.start_time = time.time()

    def to_dict(self):
        """(training rows, test rows): every epoch's ``EpochSummary.to_dict()`` plus ``total_used_time``, the time of
        all epochs up to and including it (deep500/lv2/summaries.py:54-68 builds two data frames of these rows)."""
        def rows(summaries):
            out, total = [], 0.0
            for s in summaries:
                total += s.time or 0.0
                out.append(dict(s.to_dict(), total_used_time=total))
            return out
        return rows(self.train_summaries), rows(self.test_summaries)

    def as_dict(self) -> dict:
        conv = lambda s: {"epoch": s.epoch, "loss": s.mean_loss, "accuracy": s.accuracy, "time": s.time, "lr": s.lr}
        return {"train": [conv(s) for s in self.train_summaries], "test": [conv(s) for s in self.test_summaries]}


class TerminalBarEvent(TrainingEvent):
    """Progress output on the terminal (tqdm when available)."""

    def __init__(self, stream=sys.stderr):
        self.stream, self.bar = stream, None

    def before_epoch(self, epoch, runner, training_stats):
        try:
            from tqdm import tqdm
            self.bar = tqdm(total=len(runner.train_set), desc="epoch %d" % epoch, file=self.stream, leave=False)
        except Exception:
            self.bar = None

    def after_training_step(self, executor, optimizer, outputs, loss):
        if self.bar is not None:
            self.bar.update(1)
            self.bar.set_postfix(loss="%.4f" % float(loss))

    def after_epoch(self, epoch, runner, training_stats):
        if self.bar is not None:
            self.bar.close()
        s = training_stats.current_summary(True)
        print("epoch %d: loss %.4f  train-acc %s  %.1fs" % (epoch, s.mean_loss, s.accuracy, s.time), file=self.stream)


class SummaryGeneratorEvent(TrainingEvent):
    """Fills EpochSummary objects: losses per step, accuracy and wall time per epoch."""

    def __init__(self):
        self._t = 0.0
        self.stats: Optional[TrainingStatistics] = None

    def before_training(self, runner, training_stats):
        self.stats = training_stats

    def before_epoch(self, epoch, runner, training_stats):
        self.stats = training_stats
        training_stats.train_summaries.append(EpochSummary(epoch, True))
        self._t = time.time()

    def after_training_step(self, executor, optimizer, outputs, loss):
        if self.stats is not None and self.stats.train_summaries:
            self.stats.train_summaries[-1].losses.append(float(loss))

    def after_epoch(self, epoch, runner, training_stats):
        training_stats.train_summaries[-1].time = time.time() - self._t


class SummaryGeneratorInferenceEvent(SummaryGeneratorEvent):
    """Adds the seconds spent in every forward pass and in every optimizer step to the epoch summaries
    (deep500/lv2/events/summary_generator.py:113-133).  The forward times come from the executor's own hooks, so the
    event has to be in the executor's event list as well as in the trainer's."""

    def __init__(self):
        super().__init__()
        self._fwd0 = self._opt0 = None
        self._testing = False

    def _summary(self):
        if self.stats is None:
            return None
        pool = self.stats.test_summaries if self._testing else self.stats.train_summaries
        return pool[-1] if pool else None

    def before_test_set(self, runner, training_stats, sampler):
        self.stats, self._testing = training_stats, True

    def after_test_set(self, runner, training_stats, sampler):
        self._testing = False

    def before_executor(self, inputs):
        self._fwd0 = time.perf_counter()

    def after_inference(self, outputs):
        s = self._summary()
        if s is not None and self._fwd0 is not None and not self._testing:
            s.time_used_inference.append(time.perf_counter() - self._fwd0)
        self._fwd0 = None

    def before_optimizer_step(self, executor, optimizer, inputs):
        self._opt0 = time.perf_counter()

    def after_optimizer_step(self, executor, optimizer, loss):
        s = self._summary()
        if s is not None and self._opt0 is not None:
            s.time_used_optimizing.append(time.perf_counter() - self._opt0)
        self._opt0 = None


class AccuracyAbortEvent(TrainingEvent):
    def __init__(self, target: float):
        self.target = target

    def after_test_set(self, runner, training_stats, sampler):
        acc = training_stats.test_summaries[-1].accuracy if training_stats.test_summaries else None
        if acc is not None and acc >= self.target:
            raise StopTraining("target accuracy %.4f reached" % self.target)


class TimeAbortAfterTestEvent(TrainingEvent):
    def __init__(self, seconds: float):
        self.seconds, self.t0 = seconds, None

    def before_training(self, runner, training_stats):
        self.t0 = time.time()

    def after_test_set(self, runner, training_stats, sampler):
        if time.time() - self.t0 > self.seconds:
            raise StopTraining("time budget used up")


class TimeAbortImmediateEvent(TrainingEvent):
    """Ends the run after the first optimizer step past the time budget; test passes are not cut short
    (deep500/lv2/events/stopping_conditions.py:35-47)."""

    def __init__(self, seconds: float):
        self.seconds, self.t0 = seconds, None

    def before_training(self, runner, training_stats):
        self.t0 = time.time()

    def after_training_step(self, executor, optimizer, outputs, loss):
        if time.time() - self.t0 > self.seconds:
            raise StopTraining("time budget used up")


class HyperparameterSchedule(TrainingEvent):
    """Set optimizer hyper-parameters while training, once per epoch or once per step.  Each hyper-parameter is given
    either as a function of the epoch (step) number or as a list of ``(epoch or step, value)`` pairs, which is a
    piecewise-constant schedule: the value of the last pair whose position has been reached
    (deep500/lv2/events/hyperparameter_schedule.py:8-63)."""

    def __init__(self, per_epoch: bool, **schedules):
        self.per_epoch, self.step = per_epoch, 0
        self.schedules = {}
        for name, sch in schedules.items():
            if callable(sch):
                self.schedules[name] = sch
            else:
                pairs = sorted(((int(k), v) for k, v in sch), key=lambda kv: kv[0])
                self.schedules[name] = (lambda pos, pairs=pairs: next((v for k, v in reversed(pairs) if pos >= k), None))

    def _apply(self, optimizer, position: int):
        for name, fn in self.schedules.items():
            value = fn(position)
            if value is not None:                        # a list schedule says nothing before its first position
                optimizer.set_parameter(name, value)

    def before_epoch(self, epoch, runner, training_stats):
        if self.per_epoch:
            self._apply(runner.optimizer, epoch)

    def before_optimizer_step(self, executor, optimizer, inputs):
        if not self.per_epoch:
            self._apply(optimizer, self.step)
            self.step += 1


class EpochHPSchedule(HyperparameterSchedule):
    """``EpochHPSchedule(learning_rate=lambda epoch: ...)`` or ``EpochHPSchedule(learning_rate=[(0, 0.1), (81, 0.01)])``."""

    def __init__(self, **schedules):
        super().__init__(True, **schedules)


class StepHPSchedule(HyperparameterSchedule):
    def __init__(self, **schedules):
        super().__init__(False, **schedules)


class CsvWriterEvent(TrainingEvent):
    def __init__(self, path: str, folder: Optional[str] = None):
        self.path = path if folder is None else os.path.join(folder, path)

    def after_training(self, runner, training_stats):
        with open(self.path, "w", newline="") as f:
            w = csv.writer(f)
            w.writerow(["phase", "epoch", "loss", "accuracy", "time"])
            for phase, ss in (("train", training_stats.train_summaries), ("test", training_stats.test_summaries)):
                for s in ss:
                    w.writerow([phase, s.epoch, s.mean_loss, s.accuracy, s.time])


class LossPlotGeneratorEvent(TrainingEvent):
    """Per-step loss series of every epoch (written as JSON: no plotting library here)."""

    def __init__(self, path: str, folder: Optional[str] = None):
        self.path = path if folder is None else os.path.join(folder, path)

    def after_training(self, runner, training_stats):
        with open(self.path + ".json", "w") as f:
            json.dump({"train_loss": [s.losses for s in training_stats.train_summaries]}, f)


class BoxPlotGeneratorEvent(LossPlotGeneratorEvent):
    def after_training(self, runner, training_stats):
        import numpy as np
        q = []
        for s in training_stats.train_summaries:
            if s.losses:
                a = np.asarray(s.losses)
                q.append([float(np.percentile(a, p)) for p in (0, 25, 50, 75, 100)])
        with open(self.path + ".json", "w") as f:
            json.dump({"loss_quartiles_per_epoch": q}, f)


class SaveWrongsEvent(TrainingEvent):
    """Keeps the indices of misclassified test samples of the last test pass."""

    def __init__(self):
        self.wrong: List[int] = []
        self._offset = 0

    def before_test_set(self, runner, training_stats, sampler):
        self.wrong, self._offset = [], 0

    def record(self, predictions, labels):
        import numpy as np
        bad = np.nonzero(np.asarray(predictions) != np.asarray(labels))[0]
        self.wrong.extend((bad + self._offset).tolist())
        self._offset += len(labels)
