"""Classic distributed optimizers on top of the process group.

Counterparts of deep500/frameworks/reference/distributed_optimizers.py:10-117:
ConsistentParameterServer (gather at root, mean, update, broadcast), InconsistentParameterServer
(asynchronous: the server applies gradients in arrival order), ConsistentDecentralized
(allreduce of gradients / P), ModelAverageDecentralized (local update, then allreduce of the
parameters / P) and ConsistentNeighbors (ring-neighbour averaging / 3); of the Caffe2 MPI
operators they map to (deep500/frameworks/caffe2/support/mpi_operations.cc:10-339: send, recv,
broadcast, gather, allreduce, allreduce-mean, reduce-mean); and of HorovodDistributedOptimizer
(deep500/frameworks/tensorflow/tf_distributed_optimizer.py).  Each wraps a base optimizer
from ``optim.base`` and intercepts its gradients; bulk data moves with NCCL on GPUs.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..parallel.group import Group, init as init_group
from .base import ThreeStepOptimizer


class DistributedOptimizer:
    def __init__(self, base_optimizer: ThreeStepOptimizer, group: Optional[Group] = None):
        self.base = base_optimizer
        self.executor = base_optimizer.executor
        self.network = base_optimizer.network
        self.group = group if group is not None else init_group()
        self.loss = base_optimizer.loss

    def set_parameter(self, name, value, predicate=None):
        self.base.set_parameter(name, value, predicate)

    def train(self, steps, sampler, events=()):
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

    def _backprop(self, inputs):
        self.base.new_input()
        for name, p in self.executor.module.named_parameters():
            self.base.prepare_param(name, p)
        self.executor.module.zero_grad(set_to_none=True)
        return self.executor.inference_and_backprop(inputs, self.loss)

    def _params(self):
        return [(n, p) for n, p in self.executor.module.named_parameters() if p.grad is not None]


class ConsistentDecentralized(DistributedOptimizer):
    """Synchronous allreduce of gradients, every rank applies the mean."""

    def step(self, inputs):
        out = self._backprop(inputs)
        with torch.no_grad():
            for name, p in self._params():
                g = self.group.sync_all(p.grad, average=True)
                p.copy_(self.base.update_rule(g, p, name))
        return out


class HorovodStyleOptimizer(ConsistentDecentralized):
    """One fused allreduce over all gradients (tensor fusion), otherwise as above."""

    def step(self, inputs):
        out = self._backprop(inputs)
        with torch.no_grad():
            params = self._params()
            flat = torch.cat([p.grad.reshape(-1).float() for _, p in params])
            self.group.sync_all(flat, average=True)
            off = 0
            for name, p in params:
                n = p.numel()
                p.copy_(self.base.update_rule(flat[off:off + n].view_as(p).to(p.dtype), p, name))
                off += n
        return out


class ModelAverageDecentralized(DistributedOptimizer):
    """Local update, then the parameters are averaged over all ranks."""

    def step(self, inputs):
        out = self._backprop(inputs)
        with torch.no_grad():
            for name, p in self._params():
                p.copy_(self.base.update_rule(p.grad, p, name))
                self.group.sync_all(p.data, average=True)
        return out


class ConsistentNeighbors(DistributedOptimizer):
    """Gradient averaged with the two ring neighbours (sum of three / 3)."""

    def step(self, inputs):
        out = self._backprop(inputs)
        with torch.no_grad():
            for name, p in self._params():
                g = self.group.reduce_from_neighbors(p.grad.clone()).div_(3.0)
                p.copy_(self.base.update_rule(g, p, name))
        return out


class ConsistentParameterServer(DistributedOptimizer):
    """Rank 0 gathers all gradients, applies the mean and broadcasts the parameters."""

    def step(self, inputs):
        out = self._backprop(inputs)
        g = self.group
        with torch.no_grad():
            for name, p in self._params():
                parts = g.gather_at_root(p.grad)
                if g.rank == 0:
                    mean = torch.stack(parts).float().mean(0).to(p.grad.dtype)
                    p.copy_(self.base.update_rule(mean, p, name))
                g.sync_all_with_root(p.data, 0)
        return out


class InconsistentParameterServer(DistributedOptimizer):
    """Asynchronous parameter server: workers push gradients and pull parameters without
    waiting for each other; rank 0 serves requests in arrival order.  Works with world >= 2;
    rank 0 is the server and does not train.  ``serve(num_updates)`` runs the server loop."""

    def __init__(self, base_optimizer, group=None):
        super().__init__(base_optimizer, group)
        self._names = [n for n, p in self.executor.module.named_parameters() if p.requires_grad]
        self._flat_len = sum(p.numel() for _, p in self.executor.module.named_parameters() if p.requires_grad)

    def _flat_params(self):
        return torch.cat([p.detach().reshape(-1).float() for p in self.executor.module.parameters() if p.requires_grad])

    def _load_flat(self, flat):
        off = 0
        with torch.no_grad():
            for p in self.executor.module.parameters():
                if p.requires_grad:
                    n = p.numel()
                    p.copy_(flat[off:off + n].view_as(p).to(p.dtype))
                    off += n

    def serve(self, num_updates: int):
        g = self.group
        buf = torch.empty(self._flat_len, device=g.device)
        for _ in range(num_updates):
            src = g.wait_for_any_rank(buf, tag=1)
            off = 0
            with torch.no_grad():
                for name, p in self.executor.module.named_parameters():
                    if p.requires_grad:
                        n = p.numel()
                        p.copy_(self.base.update_rule(buf[off:off + n].view_as(p).to(p.dtype), p, name))
                        off += n
            g.send_to_rank(self._flat_params(), src, tag=2)

    def step(self, inputs):
        g = self.group
        assert g.rank != 0, "rank 0 is the parameter server: call serve()"
        out = self._backprop(inputs)
        flat = torch.cat([(p.grad if p.grad is not None else torch.zeros_like(p)).reshape(-1).float()
                          for p in self.executor.module.parameters() if p.requires_grad])
        g.send_to_root(flat, tag=1)
        new = torch.empty_like(flat)
        g.wait_for_root(new, tag=2)
        self._load_flat(new)
        return out
