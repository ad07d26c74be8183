import pytest
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


def test_a_recipe_in_the_reference_form_runs(capsys):
    """FIXED / MUTABLE / METRICS as deep500/recipes/cifar10_resnet44.py writes them — model and data set by name,
    sampler class with transformations, executor factory, optimizer class with a three-argument gradient modifier,
    a list schedule, an accuracy bar in percent — shrunk to a size a CPU trains in seconds."""
    import torch
    from eagersgd_b200 import data as D
    from eagersgd_b200.optim.base import MomentumOptimizer
    from eagersgd_b200.recipes import run_recipe
    from eagersgd_b200.train import events as E, metrics as M
    from eagersgd_b200.train.executor import from_model
    from eagersgd_b200.utils.device import CPUDevice
    seen = set()

    def weight_decay(name, param, grad):
        seen.add(name)
        if "bias" in name or len(param.shape) == 1:
            return grad
        grad += 1e-4 * param
        return grad

    torch.manual_seed(0)
    fixed = {"model": "simple_mnist", "dataset": "mnist",      # (a ResNet's slow batch-norm averages need more steps than a test has)
             "dataset_kwargs": dict(synthetic_samples=256, noise=0.25), "epochs": 3}
    mutable = {"batch_size": 32, "executor": from_model, "executor_kwargs": dict(device=CPUDevice()),
               "train_sampler": D.ShuffleSampler,
               "train_sampler_kwargs": dict(seed=0, transformations=[D.Cutout(1, 4, seed=1)]),
               "validation_sampler": D.OrderedSampler,
               "optimizer": MomentumOptimizer, "optimizer_args": (0.05, 0.9), "optimizer_kwargs": dict(gradient_modifier=weight_decay),
               "events": [E.EpochHPSchedule(learning_rate=[(0, 0.05), (2, 0.01)])]}
    assert run_recipe(fixed, mutable, [(M.TestAccuracy(max_acc=True), 60.0)]) is True
    assert "PASSED" in capsys.readouterr().out and len(seen) >= 4 and any(n.endswith("bias") for n in seen)
    assert run_recipe(fixed, mutable, [(M.TestAccuracy(), 101.0)]) is False           # an unreachable bar is reported
    assert "FAIL TestAccuracy" in capsys.readouterr().out
    with pytest.raises(RuntimeError, match="overlap"):
        run_recipe(dict(fixed, batch_size=8), mutable, [])
    with pytest.raises(SyntaxError, match="Optimizer"):
        run_recipe(fixed, {k: v for k, v in mutable.items() if k != "optimizer"}, [])
