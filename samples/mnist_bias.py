"""Does a shuffling sampler visit every class equally often?  A histogram of the labels it returns.

    python samples/mnist_bias.py

Counterpart of deep500 samples/mnist_bias.py:11-19 (``DatasetBias`` metric over a ``ShuffleSampler``).
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import numpy as np  # noqa: E402

from eagersgd_b200.data import ShuffleSampler  # noqa: E402
from eagersgd_b200.train.metrics import DatasetBias  # noqa: E402
from train_mnist import synthetic_digits  # noqa: E402


def histogram(dataset, batch=10):
    sampler = ShuffleSampler(dataset, batch, seed=0)
    metric = DatasetBias(10)
    for b in sampler:
        metric.update(b["y"])
    return np.asarray(metric.measure())


def main():
    train, test = synthetic_digits(2000, 1), synthetic_digits(500, 2)
    th, vh = histogram(train), histogram(test)
    print("training set: %d samples seen, per class %s" % (th.sum(), th.astype(int).tolist()))
    print("test set:     %d samples seen, per class %s" % (vh.sum(), vh.astype(int).tolist()))
    assert th.sum() == len(train) and vh.sum() == len(test)
    return th, vh


if __name__ == "__main__":
    main()
