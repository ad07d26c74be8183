"""Learning-rate schedules of the reference run loops.

``learning_rate_with_decay``: base rate 0.1 * batch / denom, piecewise-constant decay at epoch
boundaries, optional linear warm-up over the first epochs
(official/resnet/resnet_run_loop_solo_imagenet_300.py:164-217;
ImageNet: boundaries 30/60/80/90 with factors 1, .1, .01, .001, 1e-4, 5-epoch warm-up,
imagenet_main_eagersgd.py:333-368; CIFAR-10: 81/122/164, cifar10_main.py:235-242).
"""
from __future__ import annotations

from typing import Callable, Sequence


def learning_rate_with_decay(batch_size: int, batch_denom: int, num_images: int, boundary_epochs: Sequence[int],
                             decay_rates: Sequence[float], base_lr: float = 0.1, warmup: bool = False,
                             warmup_epochs: int = 5, start_epoch: int = 0) -> Callable[[int], float]:
    """Returns ``lr(global_step)``."""
    initial = base_lr * batch_size / batch_denom
    batches_per_epoch = num_images / batch_size
    boundaries = [int(batches_per_epoch * e) for e in boundary_epochs]
    values = [initial * d for d in decay_rates]
    offset = int(start_epoch * batches_per_epoch)

    def lr(step: int) -> float:
        step = step + offset
        v = values[sum(1 for b in boundaries if step >= b)]
        if warmup:
            w = int(batches_per_epoch * warmup_epochs)
            if step < w:
                return initial * step / max(w, 1)
        return v

    return lr


# learning-rate boundaries (epochs) by --regime (imagenet_main_eagersgd.py:333-340): the full 90-epoch run and two short ones
IMAGENET_REGIMES = {0: [30, 60, 80, 90], 1: [30, 35, 39, 40], 2: [15, 20, 22, 30]}


def imagenet_schedule(batch_size: int, num_images: int = 1281167, warmup: bool = True, start_epoch: int = 0,
                      regime: int = 0):
    return learning_rate_with_decay(batch_size, 256, num_images, IMAGENET_REGIMES[regime], [1, 0.1, 0.01, 0.001, 1e-4],
                                    warmup=warmup, start_epoch=start_epoch)


def cifar10_schedule(batch_size: int, num_images: int = 50000):
    return learning_rate_with_decay(batch_size, 128, num_images, [81, 122, 164], [1, 0.1, 0.01, 0.001])
