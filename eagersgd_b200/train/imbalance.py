"""Seeded load-imbalance injectors.

All ranks draw from the same seeded stream, so they agree on who is delayed without
communicating — as in the reference, where ranks equal to either of two seeded
``randint(size)`` draws sleep 0.32 s per step
(official/resnet/resnet_run_loop_solo_imagenet_300.py:288-298) and the fflib2 evaluation
programs ``usleep`` per rank (evaluation/ssgd.c:66, rsgd_synch_recv.c:68-184).
The delay is a host sleep on CPU and a bounded spin kernel on the rank's stream on GPUs.
"""
from __future__ import annotations

import random
import time
from typing import List, Optional

import torch


class ImbalanceInjector:
    """Base: ``delay_for(step, rank)`` seconds; ``apply(rank, device)`` performs the delay."""

    def __init__(self, world: int, seed: int = 1234):
        self.world, self.rng, self.step = world, random.Random(seed), 0

    def delays(self) -> List[float]:
        """Delay of every rank for the next step (identical on all ranks)."""
        raise NotImplementedError

    def apply(self, rank: int, device: Optional[torch.device] = None) -> float:
        d = self.delays()[rank]
        self.step += 1
        if d > 0:
            if device is not None and device.type == "cuda":
                from ..parallel import _native as N
                N.check_cuda(N.cuda().esgd_spin(int(d * 1e9), torch.cuda.current_stream(device).cuda_stream),
                             "delay injection")
            else:
                time.sleep(d)
        return d


class NoImbalance(ImbalanceInjector):
    def delays(self):
        return [0.0] * self.world


class FixedRanksSleep(ImbalanceInjector):
    """``num_victims`` seeded-random ranks sleep ``seconds`` (reference: 2 draws x 0.32 s)."""

    def __init__(self, world, seconds=0.32, num_victims=2, seed=1234):
        super().__init__(world, seed)
        self.seconds, self.num_victims = seconds, num_victims

    def delays(self):
        d = [0.0] * self.world
        for _ in range(self.num_victims):
            d[self.rng.randrange(self.world)] = self.seconds
        return d


class RandomRankFactor(ImbalanceInjector):
    """One random rank is delayed by ``factor`` x the undisturbed step time."""

    def __init__(self, world, step_time, factor=1.5, seed=1234):
        super().__init__(world, seed)
        self.step_time, self.factor = step_time, factor

    def delays(self):
        d = [0.0] * self.world
        d[self.rng.randrange(self.world)] = self.factor * self.step_time
        return d


class ExponentialDelays(ImbalanceInjector):
    """``num_victims`` random ranks are delayed by Exp(mean = mean_factor x step time)."""

    def __init__(self, world, step_time, mean_factor=0.5, num_victims=2, seed=1234, cap_factor=5.0):
        super().__init__(world, seed)
        self.step_time, self.mean_factor, self.num_victims, self.cap = step_time, mean_factor, num_victims, cap_factor

    def delays(self):
        d = [0.0] * self.world
        for _ in range(self.num_victims):
            v = self.rng.randrange(self.world)
            d[v] = min(d[v] + self.rng.expovariate(1.0 / (self.mean_factor * self.step_time)),
                       self.cap * self.step_time)
        return d


class ConstantRanks(ImbalanceInjector):
    """The same ranks are slow every step (the 'constantly imbalanced' regime)."""

    def __init__(self, world, ranks=(0, 1), seconds=0.2, seed=1234):
        super().__init__(world, seed)
        self.ranks, self.seconds = tuple(ranks), seconds

    def delays(self):
        return [self.seconds if r in self.ranks else 0.0 for r in range(self.world)]
