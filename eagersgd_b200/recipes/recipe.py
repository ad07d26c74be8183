"""Declarative training recipes and their runner.

A recipe fixes the components of an experiment (model, dataset, optimizer, epochs), names the
knobs a user may change, and states the metrics it must reach — the reference's FIXED / MUTABLE /
METRICS dictionaries and ``run_recipe`` (deep500/recipe.py:37-172; recipes/cifar10_resnet44.py
with a 93 % test-accuracy bar, recipes/imagenet_resnet50.py with 75 %).
"""
from __future__ import annotations

import copy
from typing import Callable, Dict, Optional

import torch

from ..data import OrderedSampler, ShuffleSampler, SyntheticImageDataset
from ..optim.base import TorchOptimizer
from ..parallel.group import init as init_group
from ..train.events import AccuracyAbortEvent, EpochHPSchedule, SummaryGeneratorEvent, TerminalBarEvent
from ..train.executor import GraphExecutor, classification_loss
from ..train.trainer import Trainer


class Recipe:
    def __init__(self, fixed: Dict, mutable: Dict, metrics: Dict):
        self.fixed, self.mutable, self.metrics = fixed, mutable, metrics

    def with_overrides(self, **kw) -> "Recipe":
        r = copy.deepcopy(self)
        for k, v in kw.items():
            if k not in r.mutable:
                raise KeyError("%s is not a mutable component of this recipe" % k)
            r.mutable[k] = v
        return r


def run_recipe(recipe: Recipe, datasets=None, verbose: bool = True) -> Dict:
    """Build everything the recipe names, train, and check the metrics.  ``datasets`` is an optional
    (train, test) pair; without it synthetic data of the recipe's shape is used."""
    f, m = recipe.fixed, recipe.mutable
    group = init_group()
    torch.manual_seed(m.get("seed", 0))
    model = f["model"]().to(group.device)
    if datasets is None:
        train = SyntheticImageDataset(m.get("synthetic_samples", 512), f["shape"], f["classes"], seed=1)
        test = SyntheticImageDataset(128, f["shape"], f["classes"], seed=2)
    else:
        train, test = datasets
    tr = ShuffleSampler(train, m["batch_size"], seed=m.get("seed", 0))
    te = OrderedSampler(test, m["batch_size"])
    ex = GraphExecutor(model, classification_loss, events=[])
    inner = torch.optim.SGD(model.parameters(), lr=m["learning_rate"], momentum=m.get("momentum", 0.9),
                            weight_decay=m.get("weight_decay", 1e-4))
    wrap: Optional[Callable] = m.get("distributed_optimizer")
    opt = TorchOptimizer(ex, wrap(inner, group) if wrap else inner)
    events = [SummaryGeneratorEvent()]
    if verbose and group.rank == 0:
        events.append(TerminalBarEvent())
    if "lr_schedule" in m:
        events.append(EpochHPSchedule(learning_rate=m["lr_schedule"]))
    if "accuracy" in recipe.metrics:
        events.append(AccuracyAbortEvent(recipe.metrics["accuracy"]))
    stats = Trainer(tr, te, ex, opt).run_loop(int(m["epochs"]), events)
    acc = stats.test_summaries[-1].accuracy if stats.test_summaries else None
    result = {"accuracy": acc, "passed": acc is not None and acc >= recipe.metrics.get("accuracy", 0.0),
              "epochs_run": len(stats.train_summaries), "stats": stats.as_dict()}
    if hasattr(opt.opt, "close"):
        opt.opt.close()
    return result
