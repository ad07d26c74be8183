"""Declarative training recipes and their runner.

A recipe fixes the components of an experiment (model, dataset, optimizer, epochs), names the
knobs a user may change, and states the metrics it must reach — the reference's FIXED / MUTABLE /
METRICS dictionaries and ``run_recipe`` (deep500/recipe.py:37-172; recipes/cifar10_resnet44.py
with a 93 % test-accuracy bar, recipes/imagenet_resnet50.py with 75 %).
"""
from __future__ import annotations

import copy
from typing import Callable, Dict, List, Optional, Tuple

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


def run_recipe_dicts(fixed: Dict, mutable: Dict, metrics: List[Tuple]) -> bool:
    """A recipe in the reference's own form: two dictionaries of components and a list of ``(metric, acceptable value)``
    pairs (deep500/recipe.py:37-172, recipes/cifar10_resnet44.py).  Every component ``c`` other than ``batch_size``,
    ``epochs`` and ``events`` may come with ``c_args`` / ``c_kwargs``.

      * ``model``: a name for ``models.create_model`` (``'resnet'`` with ``model_kwargs=dict(depth=44)``), the path of
        an ``.onnx`` file, or a callable ``(batch_size, classes=, shape=, ...) -> torch.nn.Module``;
      * ``dataset``: a name known to ``data.dataset_shape`` (``dataset_kwargs=dict(path=...)`` to read files, synthetic
        data of its shape otherwise) or a callable ``(input_node, label_node, ...) -> (train, validation)`` with
        ``shape`` and ``loss`` attributes;
      * ``train_sampler`` / ``validation_sampler``: sampler classes (or ready samplers);
      * ``executor``: a callable on the model, e.g. ``train.executor.from_model`` (or a ready executor);
      * ``optimizer``: a class taking ``(executor, 'loss', *optimizer_args, **optimizer_kwargs)``;
      * ``epochs``, ``batch_size``, ``events``.

    Returns True when every metric with an acceptable value reaches it; prints the ones that do not."""
    import os

    from .. import data as D
    from ..graph import GraphNetwork, load_onnx
    from ..models import create_model
    from ..train.metrics import TrainingAccuracy, WallclockTime
    from ..train.trainer import test_training
    if any(k in mutable for k in fixed):
        raise RuntimeError("Fixed and mutable components cannot overlap")
    comps = dict(fixed, **mutable)
    for k in list(comps):
        if k not in ("batch_size", "epochs", "events") and not k.endswith(("_args", "_kwargs")):
            comps.setdefault(k + "_args", ())
            comps.setdefault(k + "_kwargs", {})
    for need, what in (("dataset", "Dataset"), ("model", "Model"), ("batch_size", "Batch size"), ("executor", "Executor"),
                       ("optimizer", "Optimizer"), ("epochs", "Epochs")):
        if need not in comps:
            raise SyntaxError("%s must be specified in training recipe" % what)
    ds = comps["dataset"]
    shape = D.dataset_shape(ds) if isinstance(ds, str) else ds.shape
    loss_fn = D.dataset_loss(ds) if isinstance(ds, str) else ds.loss
    classes, sample_shape = shape[0], tuple(shape[1:])
    batch = comps["batch_size"]
    model = comps["model"]
    if isinstance(model, str) and os.path.isfile(model):
        module = GraphNetwork(load_onnx(model))
    elif isinstance(model, str):
        module = create_model(model, batch, *comps["model_args"], classes=classes, shape=sample_shape, **comps["model_kwargs"])
    else:
        module = model(batch, *comps["model_args"], classes=classes, shape=sample_shape, **comps["model_kwargs"])
    input_node, label_node = "x", "y"
    if isinstance(ds, str):
        train_set, validation_set = D.load_dataset(ds, input_node, label_node, *comps["dataset_args"], **comps["dataset_kwargs"])
    else:
        train_set, validation_set = ds(input_node, label_node, *comps["dataset_args"], **comps["dataset_kwargs"])

    def sampler(key, dataset):
        if key not in comps:
            return dataset
        sm = comps[key]
        return sm if isinstance(sm, D.Sampler) else sm(dataset, batch, *comps[key + "_args"], **comps[key + "_kwargs"])
    train_sampler, validation_sampler = sampler("train_sampler", train_set), sampler("validation_sampler", validation_set)
    ex = comps["executor"]
    if not isinstance(ex, GraphExecutor):
        ex = ex(module, *comps["executor_args"], **dict(dict(loss_fn=loss_fn, data_node=input_node, label_node=label_node),
                                                        **comps["executor_kwargs"]))
    optimizer = comps["optimizer"](ex, "loss", *comps["optimizer_args"], **comps["optimizer_kwargs"])
    clock = WallclockTime(reruns=1, avg_over=1)
    import time
    t0 = time.perf_counter()
    test_training(ex, train_sampler, validation_sampler, optimizer, comps["epochs"], batch,
                  metrics=[m for m, _ in metrics], events=comps.get("events"))
    clock.times.append((time.perf_counter() - t0) * 1e3)
    ok = True
    for metric, acceptable in list(metrics) + [(clock, None)]:
        result = metric.measure()
        if acceptable is not None and acceptable > 1 and isinstance(metric, TrainingAccuracy) and result is not None:
            result = 100.0 * result               # the reference's recipes state accuracies in percent
        if acceptable is not None and (result is None or result < acceptable):
            print("FAIL %s: %s (Acceptable: %s)" % (type(metric).__name__, result, acceptable))
            ok = False
    if ok:
        print("PASSED")
    return ok


def run_recipe(recipe, datasets=None, verbose: bool = True):
    """Build everything the recipe names, train, and check the metrics.  ``datasets`` is an optional
    (train, test) pair; without it synthetic data of the recipe's shape is used.  Called with the reference's three
    arguments — ``run_recipe(FIXED, MUTABLE, METRICS)`` — it runs a recipe in that form (``run_recipe_dicts``)."""
    if isinstance(recipe, dict):
        return run_recipe_dicts(recipe, datasets, verbose)
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
