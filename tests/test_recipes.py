import torch

from eagersgd_b200.models.resnet import cifar_resnet
from eagersgd_b200.recipes import Recipe, run_recipe
from eagersgd_b200.recipes.cifar10_resnet44 import RECIPE as CIFAR
from eagersgd_b200.recipes.imagenet_resnet50 import RECIPE as IMNET


def test_recipe_declarations():
    assert CIFAR.metrics["accuracy"] == 0.93 and IMNET.metrics["accuracy"] == 0.75
    assert CIFAR.mutable["lr_schedule"](0) == 0.1 and abs(CIFAR.mutable["lr_schedule"](130) - 0.001) < 1e-9
    try:
        CIFAR.with_overrides(model=None)
        assert False
    except KeyError:
        pass


def test_run_small_recipe():
    r = Recipe(fixed={"model": lambda: cifar_resnet(8), "shape": (3, 32, 32), "classes": 10},
               mutable={"batch_size": 16, "epochs": 1, "learning_rate": 0.05, "synthetic_samples": 64,
                        "distributed_optimizer": None, "seed": 0},
               metrics={})
    out = run_recipe(r, verbose=False)
    assert out["passed"] and out["epochs_run"] == 1 and 0.0 <= out["accuracy"] <= 1.0
