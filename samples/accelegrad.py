"""Define a new optimizer from three small methods and train with it: AcceleGrad.

    python samples/accelegrad.py [--epochs 2]

Kfir Y. Levy, Alp Yurtsever, Volkan Cevher, "Online Adaptive Methods, Universality and Acceleration",
NeurIPS 2018.  The reference ships the same example on its three-step optimizer interface
(deep500 samples/accelegrad.py:5-66): ``new_input`` once per step, ``prepare_param`` before the gradient
is computed, ``update_rule`` after.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch  # noqa: E402

from eagersgd_b200.data import OrderedSampler, ShuffleSampler  # noqa: E402
from eagersgd_b200.models.small import MnistNet  # noqa: E402
from eagersgd_b200.optim.base import ThreeStepOptimizer  # noqa: E402
from eagersgd_b200.train import events as E  # noqa: E402
from eagersgd_b200.train.executor import GraphExecutor, classification_loss  # noqa: E402
from eagersgd_b200.train.trainer import Trainer  # noqa: E402
from train_mnist import synthetic_digits  # noqa: E402


class AcceleGradOptimizer(ThreeStepOptimizer):
    def __init__(self, executor, loss="loss", G=0.0, D=1.0, eps=1e-6):
        super().__init__(executor, loss)
        self.G, self.D, self.eps = G, D, eps
        self.squares, self.z, self.y = {}, {}, {}
        self.t = -1

    def new_input(self):
        self.t += 1
        self.alpha_t = 1.0 if self.t <= 2 else 0.25 * (self.t + 1)
        self.tau_t = 1.0 / self.alpha_t

    def prepare_param(self, name, param):
        if name not in self.y:
            self.y[name], self.z[name], self.squares[name] = param.detach().clone(), param.detach().clone(), 0.0
        with torch.no_grad():           # the gradient is taken at x_t = tau z_t + (1 - tau) y_t
            param.copy_(self.tau_t * self.z[name] + (1.0 - self.tau_t) * self.y[name])

    def update_rule(self, grad, old_param, name):
        self.squares[name] += self.alpha_t ** 2 * float(grad.norm()) ** 2
        eta = 2.0 * self.D / (self.G ** 2 + self.squares[name] + self.eps) ** 0.5
        self.z[name] = self.z[name] - self.alpha_t * eta * grad
        self.y[name] = old_param - eta * grad
        return self.y[name]


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--epochs", type=int, default=2)
    ap.add_argument("--train-size", type=int, default=2048)
    args = ap.parse_args(argv)
    torch.manual_seed(0)
    ex = GraphExecutor(MnistNet(), classification_loss)
    trainer = Trainer(ShuffleSampler(synthetic_digits(args.train_size, 1), 64, seed=0),
                      OrderedSampler(synthetic_digits(512, 2), 128), ex, AcceleGradOptimizer(ex, D=3.0))
    stats = trainer.run_loop(args.epochs, [E.SummaryGeneratorEvent()])
    print("AcceleGrad: test accuracy after %d epochs: %.3f" % (args.epochs, stats.test_summaries[-1].accuracy))
    return stats.test_summaries[-1].accuracy


if __name__ == "__main__":
    main()
