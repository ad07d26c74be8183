"""ResNet-44 on CIFAR-10, 93 % test accuracy (deep500 recipes/cifar10_resnet44.py:47-49)."""
from ..models.resnet import cifar_resnet
from ..optim.eager import SoloAllreduceOptimizer
from .recipe import Recipe

RECIPE = Recipe(
    fixed={"model": lambda: cifar_resnet(44), "shape": (3, 32, 32), "classes": 10, "dataset": "cifar10"},
    mutable={"batch_size": 128, "epochs": 190, "learning_rate": 0.1, "momentum": 0.9, "weight_decay": 2e-4,
             "lr_schedule": lambda e: 0.1 * (0.1 ** sum(e >= b for b in (81, 122, 164))),
             "distributed_optimizer": lambda opt, group: SoloAllreduceOptimizer(opt, group, limiter=32), "seed": 0},
    metrics={"accuracy": 0.93})
