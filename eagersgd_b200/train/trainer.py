"""Trainer: epochs of optimizer steps with a test pass after each, driven by events.

Counterpart of deep500/lv2/trainer.py:22-127 (``Trainer.run_loop(epochs, events)`` with
``_train`` / ``_test_accuracy``) and of the validation helper ``test_training``
(deep500/lv2/validation/training.py:10-86).
"""
from __future__ import annotations

import time
from typing import Optional, Sequence

import numpy as np

from .events import EpochSummary, StopTraining, SummaryGeneratorEvent, TrainingStatistics


def _nothing(*a, **k):
    return None


def DefaultTrainerEvents(epochs: int = 0, stream=None):
    """What a run shows when no events are named: the progress bar on the terminal (deep500/lv2/trainer.py:18-19)."""
    import sys

    from .events import TerminalBarEvent
    return [TerminalBarEvent(stream or sys.stderr)]


class Trainer:
    def __init__(self, training_sampler, validation_sampler, executor, optimizer, output_node: str = "output",
                 network_output: str = "output"):
        self.train_set, self.test_set = training_sampler, validation_sampler
        self.executor, self.optimizer = executor, optimizer
        self.output_node = output_node

    def _accuracy(self, sampler, stats: TrainingStatistics, events, epoch: int) -> Optional[float]:
        if sampler is None:
            return None
        for e in events:
            e.before_test_set(self, stats, sampler)
        correct = total = 0
        summary = EpochSummary(epoch, False)
        sampler.reset()
        t0 = time.time()
        while True:
            batch = sampler()
            if batch is None:
                break
            for e in events:
                e.before_test_step(self.executor, batch)
                getattr(e, "before_test_batch", _nothing)(self, stats, batch)
            out = self.executor.inference(batch)
            pred = out["output"].float().argmax(-1).cpu().numpy()
            labels = np.asarray(batch[self.executor.label_node])
            correct += int((pred == labels).sum())
            total += len(labels)
            if "loss" in out:
                summary.losses.append(float(out["loss"]))
            for e in events:
                if hasattr(e, "record"):
                    e.record(pred, labels)
                e.after_test_step(self.executor, out)
                getattr(e, "after_test_batch", _nothing)(self, stats, out)
        summary.accuracy = correct / max(total, 1)
        summary.time = time.time() - t0
        stats.test_summaries.append(summary)
        for e in events:
            e.after_test_set(self, stats, sampler)
        return summary.accuracy

    def _train_epoch(self, epoch: int, stats: TrainingStatistics, events):
        self.train_set.reset()
        correct = total = 0
        while True:
            batch = self.train_set()
            if batch is None:
                break
            for e in events:
                e.before_training_step(self.executor, self.optimizer, batch)
                e.before_optimizer_step(self.executor, self.optimizer, batch)
            out = self.optimizer.step(batch)
            loss = float(out["loss"])
            if "output" in out and self.executor.label_node in batch:
                pred = out["output"].detach().float().argmax(-1).cpu().numpy()
                labels = np.asarray(batch[self.executor.label_node])
                correct += int((pred == labels).sum())
                total += len(labels)
            for e in events:
                e.after_optimizer_step(self.executor, self.optimizer, loss)
                e.after_training_step(self.executor, self.optimizer, out, loss)
        if stats.train_summaries and total:
            stats.train_summaries[-1].accuracy = correct / total

    def run_loop(self, epochs: int, events: Optional[Sequence] = None, collect_all_times: bool = False
                 ) -> TrainingStatistics:
        events = list(events or [])
        if not any(isinstance(e, SummaryGeneratorEvent) for e in events):
            events.insert(0, SummaryGeneratorEvent())
        stats = TrainingStatistics()
        try:
            for e in events:
                e.before_training(self, stats)
            self._accuracy(self.test_set, stats, events, -1)
            for epoch in range(epochs):
                for e in events:
                    e.before_epoch(epoch, self, stats)
                    getattr(e, "before_training_set", _nothing)(self, stats, self.train_set)
                self._train_epoch(epoch, stats, events)
                for e in events:
                    getattr(e, "after_training_set", _nothing)(self, stats)
                    e.after_epoch(epoch, self, stats)
                self._accuracy(self.test_set, stats, events, epoch)
        except StopTraining:
            pass
        for e in events:
            e.after_training(self, stats)
        return stats


def test_training(executor, training_set, validation_set, optimizer, epochs: int = 1, batch_size: int = 64,
                  output_node: Optional[str] = None, metrics: Optional[Sequence] = None, events: Optional[Sequence] = None
                  ) -> TrainingStatistics:
    """Train for ``epochs`` and return the statistics (deep500 ``d5.test_training``, lv2/validation/training.py:10-86).
    ``training_set`` / ``validation_set`` are samplers, or data sets, which are then drawn from in shuffled (training)
    and sequential (validation) batches of ``batch_size``.  ``metrics`` that are events (``TestAccuracy`` ...) ride along
    with ``events``; their ``measure()`` holds the result afterwards."""
    from ..data.sampler import OrderedSampler, ShuffleSampler
    if isinstance(batch_size, (list, tuple)):                # the events given as the sixth positional argument
        events, batch_size = batch_size, 64
    if training_set is not None and not callable(training_set):
        training_set = ShuffleSampler(training_set, batch_size)
    if validation_set is not None and not callable(validation_set):
        validation_set = OrderedSampler(validation_set, batch_size)
    trainer = Trainer(training_set, validation_set, executor, optimizer, **({"output_node": output_node} if output_node else {}))
    return trainer.run_loop(epochs, list(events or []) + [m for m in (metrics or []) if hasattr(m, "after_training")])
