"""Optimizer abstractions over an executor, and the classic update rules.

Counterparts of deep500/lv2/optimizer.py:13-173 (Optimizer, FirstOrderOptimizer with its
event-driven ``train`` loop, ThreeStepOptimizer {new_input, prepare_param, update_rule},
UpdateRuleOptimizer, the ``gradient_modifier`` hook), of the numpy reference rules
deep500/frameworks/reference/optimizers.py:7-123 (GradientDescent, Momentum, Adam, AdaGrad)
and of deep500/frameworks/pytorch/pytorch_optimizers.py (thin wrappers over torch.optim).
The update rules run on torch tensors, on whichever device the parameters live.
"""
from __future__ import annotations

import inspect
from typing import Callable, Dict, Optional

import torch



class Optimizer:
    def __init__(self, executor, loss: str = "loss", gradient_modifier: Optional[Callable] = None):
        self.executor, self.loss = executor, loss
        self.network = executor.network
        # (name, grad) -> grad, or the reference's (name, parameter, grad) -> grad (deep500/lv2/optimizer.py:16-31)
        self.gradient_modifier = gradient_modifier
        self.hyper: Dict[str, float] = {}

    def _modify(self, name: str, param, grad):
        """The gradient a step uses: what the ``gradient_modifier`` makes of it, if there is one."""
        fn = self.gradient_modifier
        if fn is None:
            return grad
        try:
            three = len([q for q in inspect.signature(fn).parameters.values()
                         if q.kind in (q.POSITIONAL_ONLY, q.POSITIONAL_OR_KEYWORD)]) >= 3
        except (TypeError, ValueError):
            three = False
        if not three:
            return fn(name, grad)
        with torch.no_grad():                   # such modifiers may update the gradient in place (grad += wd * param)
            return fn(name, param, grad)

    def set_parameter(self, name: str, value, predicate=None):
        self.hyper[name] = value

    def step(self, inputs) -> dict:
        raise NotImplementedError

    def train(self, steps: int, sampler, events=()):
        """Run ``steps`` optimizer steps drawing batches from ``sampler``."""
        for _ in range(steps):
            batch = sampler()
            if batch is None:
                break
            for e in events:
                e.before_optimizer_step(self.executor, self, batch)
            out = self.step(batch)
            for e in events:
                e.after_optimizer_step(self.executor, self, out.get(self.loss))
        return self


class FirstOrderOptimizer(Optimizer):
    """Gradient-based optimizer: backprop, then an update per parameter."""

    def _grads(self):
        for name, p in self.executor.module.named_parameters():
            if p.grad is None:
                continue
            yield name, p, self._modify(name, p, p.grad)


class ThreeStepOptimizer(FirstOrderOptimizer):
    """new_input() once per step, prepare_param() before backprop, update_rule() after."""

    def new_input(self): ...

    def prepare_param(self, name: str, param: torch.Tensor): ...

    def update_rule(self, grad: torch.Tensor, old_param: torch.Tensor, name: str) -> torch.Tensor:
        raise NotImplementedError

    def step(self, inputs):
        self.new_input()
        for name, p in self.executor.module.named_parameters():
            self.prepare_param(name, p)
        self.executor.module.zero_grad(set_to_none=True)
        out = self.executor.inference_and_backprop(inputs, self.loss)
        with torch.no_grad():
            for name, p, g in self._grads():
                p.copy_(self.update_rule(g, p, name))
        return out


UpdateRuleOptimizer = ThreeStepOptimizer


class GradientDescent(ThreeStepOptimizer):
    def __init__(self, executor, loss="loss", learning_rate=0.1, **kw):
        super().__init__(executor, loss, **kw)
        self.hyper["learning_rate"] = learning_rate

    def update_rule(self, grad, old_param, name):
        return old_param - self.hyper["learning_rate"] * grad.to(old_param.dtype)


class MomentumOptimizer(ThreeStepOptimizer):
    """acc = m*acc + g ; p -= lr*acc (reference optimizers.py:39-46)."""

    def __init__(self, executor, loss="loss", learning_rate=0.1, momentum=0.9, weight_decay=0.0, **kw):
        super().__init__(executor, loss, **kw)
        self.hyper.update(learning_rate=learning_rate, momentum=momentum, weight_decay=weight_decay)
        self.acc: Dict[str, torch.Tensor] = {}

    def update_rule(self, grad, old_param, name):
        g = grad.float() + self.hyper["weight_decay"] * old_param.float()
        acc = self.acc.get(name)
        acc = g.clone() if acc is None else acc.mul_(self.hyper["momentum"]).add_(g)
        self.acc[name] = acc
        return (old_param.float() - self.hyper["learning_rate"] * acc).to(old_param.dtype)


class AdamOptimizer(ThreeStepOptimizer):
    def __init__(self, executor, loss="loss", learning_rate=1e-3, beta1=0.9, beta2=0.999, epsilon=1e-8, **kw):
        super().__init__(executor, loss, **kw)
        self.hyper.update(learning_rate=learning_rate, beta1=beta1, beta2=beta2, epsilon=epsilon)
        self.t = 0
        self.m: Dict[str, torch.Tensor] = {}
        self.v: Dict[str, torch.Tensor] = {}

    def new_input(self):
        self.t += 1

    def update_rule(self, grad, old_param, name):
        h = self.hyper
        g = grad.float()
        m = self.m.get(name, torch.zeros_like(g)).mul_(h["beta1"]).add_(g, alpha=1 - h["beta1"])
        v = self.v.get(name, torch.zeros_like(g)).mul_(h["beta2"]).addcmul_(g, g, value=1 - h["beta2"])
        self.m[name], self.v[name] = m, v
        mhat = m / (1 - h["beta1"] ** self.t)
        vhat = v / (1 - h["beta2"] ** self.t)
        return (old_param.float() - h["learning_rate"] * mhat / (vhat.sqrt() + h["epsilon"])).to(old_param.dtype)


class AdaGradOptimizer(ThreeStepOptimizer):
    def __init__(self, executor, loss="loss", learning_rate=0.01, epsilon=1e-8, **kw):
        super().__init__(executor, loss, **kw)
        self.hyper.update(learning_rate=learning_rate, epsilon=epsilon)
        self.sq: Dict[str, torch.Tensor] = {}

    def update_rule(self, grad, old_param, name):
        g = grad.float()
        sq = self.sq.get(name, torch.zeros_like(g)).addcmul_(g, g)
        self.sq[name] = sq
        return (old_param.float() - self.hyper["learning_rate"] * g / (sq.sqrt() + self.hyper["epsilon"])).to(
            old_param.dtype)


class RMSPropOptimizer(ThreeStepOptimizer):
    """sq = d*sq + (1-d)*g^2 ; p -= lr * g / (sqrt(sq) + eps)  (the RMSProp of the reference's
    PyTorch backend, deep500/frameworks/pytorch/pytorch_optimizers.py)."""

    def __init__(self, executor, loss="loss", learning_rate=1e-3, decay=0.9, epsilon=1e-8, **kw):
        super().__init__(executor, loss, **kw)
        self.hyper.update(learning_rate=learning_rate, decay=decay, epsilon=epsilon)
        self.sq: Dict[str, torch.Tensor] = {}

    def update_rule(self, grad, old_param, name):
        h = self.hyper
        g = grad.float()
        sq = self.sq.get(name, torch.zeros_like(g)).mul_(h["decay"]).addcmul_(g, g, value=1 - h["decay"])
        self.sq[name] = sq
        return (old_param.float() - h["learning_rate"] * g / (sq.sqrt() + h["epsilon"])).to(old_param.dtype)


class TorchOptimizer(FirstOrderOptimizer):
    """Any ``torch.optim`` optimizer (or one of this package's eager-SGD wrappers around it)
    driven through the executor, with the ``gradient_modifier`` hook applied before the step."""

    def __init__(self, executor, torch_optimizer, loss="loss", **kw):
        super().__init__(executor, loss, **kw)
        self.opt = torch_optimizer

    def set_parameter(self, name, value, predicate=None):
        super().set_parameter(name, value)
        key = {"learning_rate": "lr"}.get(name, name)
        for g in self.opt.param_groups:
            if key in g:
                g[key] = value

    def step(self, inputs):
        self.opt.zero_grad()
        out = self.executor.inference_and_backprop(inputs, self.loss)
        if self.gradient_modifier is not None:
            with torch.no_grad():
                for name, p, g in self._grads():
                    if g is not p.grad:
                        p.grad.copy_(g)
        self.opt.step()
        return out


class LBFGSOptimizer(TorchOptimizer):
    """``torch.optim.LBFGS`` through the executor: one ``step`` evaluates the loss and its gradients as often as the
    line search asks (deep500/frameworks/pytorch/pytorch_optimizers.py:136-152)."""

    def __init__(self, executor, loss="loss", learning_rate: float = 1.0, max_iter: int = 20, max_eval: Optional[int] = None,
                 tolerance_grad: float = 1e-5, tolerance_change: float = 1e-9, history_size: int = 100, line_search_fn=None):
        params = [p for p in executor.module.parameters() if p.requires_grad]
        super().__init__(executor, torch.optim.LBFGS(params, lr=learning_rate, max_iter=max_iter, max_eval=max_eval,
                                                     tolerance_grad=tolerance_grad, tolerance_change=tolerance_change,
                                                     history_size=history_size, line_search_fn=line_search_fn), loss)
        self.evaluations = 0

    def step(self, inputs):
        last = {}

        def closure():
            self.opt.zero_grad()
            out = self.executor.inference_and_backprop(inputs, self.loss)
            if self.gradient_modifier is not None:
                with torch.no_grad():
                    for name, p, g in self._grads():
                        if g is not p.grad:
                            p.grad.copy_(g)
            self.evaluations += 1
            if not last:
                last.update(out)                         # what the step started from, like the other optimizers return
            return out[self.loss]

        self.opt.step(closure)
        return last
