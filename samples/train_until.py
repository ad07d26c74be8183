"""Train until a test accuracy is reached (or a maximum number of epochs): stopping conditions as events.

    python samples/train_until.py [ACCURACY_PERCENT] [--max-epochs 10]

Counterpart of the reference's deep500 samples/train_until.py:44-52 (DefaultTrainerEvents + AccuracyAbortEvent).
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch  # noqa: E402

from eagersgd_b200.data import OrderedSampler, ShuffleSampler  # noqa: E402
from eagersgd_b200.models.small import MnistNet  # noqa: E402
from eagersgd_b200.optim import base  # noqa: E402
from eagersgd_b200.train import events as E  # noqa: E402
from eagersgd_b200.train.executor import GraphExecutor, classification_loss  # noqa: E402
from eagersgd_b200.train.trainer import Trainer  # noqa: E402
from train_mnist import synthetic_digits  # noqa: E402


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("accuracy", nargs="?", type=float, default=90.0, help="desired test accuracy in percent")
    ap.add_argument("--max-epochs", type=int, default=10)
    ap.add_argument("--train-size", type=int, default=2048)
    args = ap.parse_args(argv)
    torch.manual_seed(0)
    ex = GraphExecutor(MnistNet(), classification_loss)
    opt = base.MomentumOptimizer(ex, learning_rate=0.05)
    trainer = Trainer(ShuffleSampler(synthetic_digits(args.train_size, 1), 64, seed=0),
                      OrderedSampler(synthetic_digits(512, 2), 128), ex, opt)
    events = [E.SummaryGeneratorEvent(), E.AccuracyAbortEvent(args.accuracy / 100.0)]
    stats = trainer.run_loop(args.max_epochs, events)
    done = len(stats.test_summaries)
    print("stopped after %d test passes at accuracy %.3f (target %.3f, at most %d epochs)"
          % (done, stats.test_summaries[-1].accuracy, args.accuracy / 100.0, args.max_epochs))
    return done


if __name__ == "__main__":
    main()
