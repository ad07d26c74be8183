"""Train a small classifier with the Trainer / events / update-rule optimizer stack.

    python samples/train_mnist.py [--epochs 3] [--optimizer MomentumOptimizer]

Uses MNIST-shaped synthetic digits (class templates plus noise; there is no network to download
the real set) so that accuracy is meaningful; the counterpart of the reference's
deep500 samples/train_mnist.py and custom_optimizer tutorial.
"""
import argparse
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from eagersgd_b200.data import NumpyDataset, OrderedSampler, ShuffleSampler  # noqa: E402
from eagersgd_b200.models.small import MnistNet  # noqa: E402
from eagersgd_b200.optim import base  # noqa: E402
from eagersgd_b200.train import events as E  # noqa: E402
from eagersgd_b200.train.executor import GraphExecutor, classification_loss  # noqa: E402
from eagersgd_b200.train.trainer import Trainer  # noqa: E402


def synthetic_digits(n, seed):
    rng = np.random.RandomState(seed)
    templates = np.random.RandomState(7).rand(10, 1, 28, 28).astype(np.float32)
    y = rng.randint(0, 10, n).astype(np.int64)
    x = templates[y] + 0.5 * rng.randn(n, 1, 28, 28).astype(np.float32)
    return NumpyDataset(x, "x", y, "y")


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--epochs", type=int, default=2)
    ap.add_argument("--optimizer", default="MomentumOptimizer")
    ap.add_argument("--train-size", type=int, default=2048)
    args = ap.parse_args(argv)
    torch.manual_seed(0)
    train, test = synthetic_digits(args.train_size, 1), synthetic_digits(512, 2)
    ex = GraphExecutor(MnistNet(), classification_loss)
    opt = getattr(base, args.optimizer)(ex, learning_rate=0.05)
    trainer = Trainer(ShuffleSampler(train, 64, seed=0), OrderedSampler(test, 128), ex, opt)
    stats = trainer.run_loop(args.epochs, [E.SummaryGeneratorEvent(), E.EpochHPSchedule(learning_rate=lambda e: 0.05 * 0.5 ** e)])
    acc = stats.test_summaries[-1].accuracy
    print("test accuracy after %d epochs: %.3f" % (args.epochs, acc))
    return acc


if __name__ == "__main__":
    main()
