"""ResNet-50 on ImageNet, 75 % top-1 (deep500 recipes/imagenet_resnet50.py:41-43)."""
from ..models.resnet import imagenet_resnet
from ..optim.eager import SoloAllreduceOptimizer
from .recipe import Recipe

RECIPE = Recipe(
    fixed={"model": lambda: imagenet_resnet(50, 1, 1001), "shape": (3, 224, 224), "classes": 1001,
           "dataset": "imagenet"},
    mutable={"batch_size": 256, "epochs": 90, "learning_rate": 0.1, "momentum": 0.9, "weight_decay": 1e-4,
             "lr_schedule": lambda e: 0.1 * (0.1 ** sum(e >= b for b in (30, 60, 80))),
             "distributed_optimizer": lambda opt, group: SoloAllreduceOptimizer(opt, group, limiter=32), "seed": 0},
    metrics={"accuracy": 0.75})
