"""Validation harnesses for operators, executors, optimizers and samplers.

``test_op_forward`` compares an operator's outputs with reference outputs under a set of metrics;
``test_op_gradient`` compares its analytic gradients with a central-difference numerical Jacobian
(deep500/lv0/validation/forward.py, gradient.py:114-157); ``test_executor_*`` do the same for whole
networks (deep500/lv1/validation/executor.py); ``test_optimizer`` / ``test_sampler`` time and
sanity-check those components (deep500/lv2/validation/optimizer.py, sampler.py).
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence

import numpy as np
import torch

from ..train.metrics import DatasetBias, L2Error, MaxError, TestMetric, WallclockTime


def DefaultOpMetrics() -> List[TestMetric]:
    """The metrics an operator test reports when none are named (deep500/lv0/validation/metrics.py:4-9)."""
    from ..train.metrics import DiffHeatmap
    return [L2Error(), MaxError(), DiffHeatmap(), WallclockTime()]


def DefaultOptimizerMetrics() -> List[TestMetric]:
    """deep500/lv2/validation/optimizer.py:8-9."""
    return [L2Error(), WallclockTime()]


def DefaultTrainingMetrics() -> List[TestMetric]:
    """deep500/lv2/validation/metrics.py:9-10."""
    from ..train.metrics import TestAccuracy, TrainingAccuracy
    return [TrainingAccuracy(), TestAccuracy()]


def _as_list(x):
    return list(x) if isinstance(x, (tuple, list)) else [x]


def test_op_forward(op: Callable, inputs: Sequence[torch.Tensor], reference_outputs, metrics: Optional[List[TestMetric]] = None,
                    rtol: float = 1e-4, atol: float = 1e-5) -> Dict[str, float]:
    outs = _as_list(op(*inputs))
    refs = _as_list(reference_outputs)
    res = {}
    for i, (o, r) in enumerate(zip(outs, refs)):
        r = torch.as_tensor(r).to(o.device)
        for m in (metrics or [L2Error(), MaxError()]):
            res["%s[%d]" % (type(m).__name__, i)] = m.measure(inputs, o, r)
        if not torch.allclose(o.float(), r.float(), rtol=rtol, atol=atol):
            raise AssertionError("forward output %d differs: max error %g" % (i, (o.float() - r.float()).abs().max()))
    return res


def numerical_jacobian(op: Callable, inputs: Sequence[torch.Tensor], wrt: int, eps: float = 1e-3) -> torch.Tensor:
    """d out / d inputs[wrt] by central differences, shape [out.numel(), in.numel()] (float64)."""
    xs = [t.detach().clone().double() for t in inputs]
    x = xs[wrt]
    flat = x.view(-1)
    out0 = _as_list(op(*[t.to(inputs[k].dtype) for k, t in enumerate(xs)]))[0]
    J = torch.zeros(out0.numel(), flat.numel(), dtype=torch.float64)
    for j in range(flat.numel()):
        old = flat[j].item()
        flat[j] = old + eps
        plus = _as_list(op(*[t.to(inputs[k].dtype) for k, t in enumerate(xs)]))[0].double().reshape(-1)
        flat[j] = old - eps
        minus = _as_list(op(*[t.to(inputs[k].dtype) for k, t in enumerate(xs)]))[0].double().reshape(-1)
        flat[j] = old
        J[:, j] = ((plus - minus) / (2 * eps)).cpu()
    return J


def test_op_gradient(op: Callable, inputs: Sequence[torch.Tensor], eps: float = 1e-3, rtol: float = 1e-2,
                     atol: float = 1e-3, wrt: Optional[Sequence[int]] = None) -> Dict[str, float]:
    """Analytic vs numerical Jacobian for every (floating) input in ``wrt``."""
    res = {}
    idx = wrt if wrt is not None else [i for i, t in enumerate(inputs) if t.is_floating_point()]
    for i in idx:
        xs = [t.detach().clone().requires_grad_(k == i) for k, t in enumerate(inputs)]
        out = _as_list(op(*xs))[0]
        J = torch.zeros(out.numel(), xs[i].numel(), dtype=torch.float64)
        for r in range(out.numel()):
            g = torch.zeros_like(out).reshape(-1)
            g[r] = 1
            (gi,) = torch.autograd.grad(out, xs[i], g.view_as(out), retain_graph=True)
            J[r] = gi.double().reshape(-1).cpu()
        Jn = numerical_jacobian(op, inputs, i, eps)
        err = (J - Jn).abs().max().item()
        res["input%d_max_error" % i] = err
        if not torch.allclose(J, Jn, rtol=rtol, atol=atol):
            raise AssertionError("gradient w.r.t. input %d differs from finite differences: %g" % (i, err))
    return res


def test_executor_inference(executor, batch, reference_output, rtol=1e-4, atol=1e-5):
    out = executor.inference(batch)["output"]
    ref = torch.as_tensor(reference_output).to(out.device)
    assert torch.allclose(out.float(), ref.float(), rtol=rtol, atol=atol)
    return {"max_error": (out.float() - ref.float()).abs().max().item()}


def test_executor_backprop(executor, batch, reference_grads: Dict[str, np.ndarray], rtol=1e-3, atol=1e-5):
    executor.module.zero_grad(set_to_none=True)
    executor.inference_and_backprop(batch)
    res = {}
    for name, ref in reference_grads.items():
        g = executor.network.fetch_gradient(name)
        res[name] = float(np.abs(g - ref).max())
        assert np.allclose(g, ref, rtol=rtol, atol=atol), name
    return res


class OneInputDataset:
    """A data set of one batch that is handed out again and again: what ``test_optimizer`` makes of a plain dictionary
    of inputs, or of an (inputs, labels) pair (deep500/lv2/validation/optimizer.py:11-27)."""

    def __init__(self, inputs: Dict[str, np.ndarray], labels: Optional[Dict[str, np.ndarray]] = None):
        self.batch = dict(inputs)
        self.batch.update(labels or {})
        names = list(inputs)
        self.data_node = names[0] if names else "x"
        self.label_node = next(iter(labels), "y") if labels else "y"

    def __len__(self):
        return 1

    def __getitem__(self, index):
        return self.batch


class _OneBatchSampler:
    def __init__(self, dataset: OneInputDataset):
        self.dataset, self.batch_size = dataset, 1

    def __call__(self):
        return self.dataset[0]

    def reset(self): ...


def test_optimizer(optimizer, sampler, steps: int = 10, device: Optional[torch.device] = None,
                   expected_params=None, rtol: float = 1e-4, atol: float = 1e-6) -> Dict[str, float]:
    """Run ``steps`` steps; returns the median step time (ms) and the loss trajectory ends.

    ``sampler`` may be a sampler, a data set (batches of one sample are drawn from it in order), a dictionary of
    input arrays, or an (inputs, labels) pair of dictionaries.  With ``expected_params`` (name -> array, or a list in
    parameter order) exactly one step is taken and the parameters are compared with them: the L2 distance per
    parameter is returned and a mismatch raises (deep500/lv2/validation/optimizer.py:29-93)."""
    if isinstance(sampler, dict):
        sampler = _OneBatchSampler(OneInputDataset(sampler))
    elif isinstance(sampler, tuple) and len(sampler) == 2 and all(isinstance(d, dict) for d in sampler):
        sampler = _OneBatchSampler(OneInputDataset(*sampler))
    elif not callable(sampler):
        if not (hasattr(sampler, "__len__") and hasattr(sampler, "__getitem__")):
            raise ValueError("test_optimizer takes a sampler, a data set, a dictionary of inputs or an (inputs, labels) pair")
        from ..data.sampler import OrderedSampler
        sampler = OrderedSampler(sampler, 1)
    if expected_params is not None:
        batch = sampler()
        out = optimizer.step(batch)
        net = optimizer.executor.network
        names = net.get_params()
        expect = expected_params if isinstance(expected_params, dict) else dict(zip(names, expected_params))
        res = {"loss": float(out["loss"])}
        for name, ref in expect.items():
            got = net.fetch_tensor(name)
            res[name] = L2Error().measure(None, got, np.asarray(ref))
            if not np.allclose(got, np.asarray(ref), rtol=rtol, atol=atol):
                raise AssertionError("parameter %s after one step differs from the expected value: L2 distance %g" % (name, res[name]))
        return res
    losses = []
    timer = WallclockTime(reruns=1, avg_over=1, device=device)

    def one():
        batch = sampler()
        if batch is None:
            sampler.reset()
            batch = sampler()
        losses.append(float(optimizer.step(batch)["loss"]))
    timer.reruns = steps
    ms = timer.time_callable(one, warmup=1)
    return {"median_step_ms": ms, "first_loss": losses[0], "last_loss": losses[-1]}


def test_sampler(sampler, batches: int = 10, expected_output=None, metrics: Optional[List[TestMetric]] = None,
                 events: Optional[Sequence] = None):
    """Draw ``batches`` batches and report the median time per batch and how many distinct sample shapes came out.

    With ``metrics`` (and optionally ``events``) it is the reference's harness: metrics that have sampler hooks
    (``before_sampling`` / ``after_sampling`` — ``SamplerEventMetric``, ``DatasetBias``) are attached to the sampler
    for the duration, every metric's ``begin`` / ``end`` brackets the draws (``reruns`` of them, at least ``batches``
    when the metric has no ``reruns``), and the list of ``measure(sampler, last batch, expected_output)`` results is
    returned (deep500/lv2/validation/sampler.py:6-66)."""
    import time
    if metrics is not None:
        attached = [m for m in metrics if hasattr(type(m), "before_sampling") or hasattr(type(m), "after_sampling")]
        attached += [e for e in (events or []) if e not in attached]
        sampler.events.extend(attached)
        last = None
        try:
            for m in metrics:
                m.begin(sampler)
            for _ in range(max([int(getattr(m, "reruns", 0) or 0) for m in metrics] + [batches])):
                last = sampler()
                if last is None:
                    sampler.reset()
                    last = sampler()
                for m in metrics:
                    if isinstance(m, DatasetBias):               # the histogram of the labels that were drawn
                        m.update(last[getattr(sampler.dataset, "label_node", "y")])
            for m in metrics:
                m.end(last)
        finally:
            if attached:
                del sampler.events[-len(attached):]
        return [m.measure(sampler, last, expected_output) for m in metrics]
    t = []
    shapes = set()
    for _ in range(batches):
        t0 = time.perf_counter()
        b = sampler()
        if b is None:
            sampler.reset()
            b = sampler()
        t.append(time.perf_counter() - t0)
        shapes.add(tuple(np.asarray(b[sampler.dataset.data_node]).shape[1:]) if hasattr(sampler.dataset, "data_node") else ())
    return {"median_batch_ms": float(np.median(t) * 1e3), "distinct_sample_shapes": len(shapes)}


for _f in (test_op_forward, test_op_gradient, test_executor_inference, test_executor_backprop, test_optimizer,
           test_sampler):
    _f.__test__ = False   # library functions, not pytest tests
