"""Hyperplane regression: y = w*·x + eps, the smallest eager-SGD workload.

fp32 linear model, x ~ N(0,1) of dimension ``dim``, a fixed teacher ``w*`` drawn
from the seed, eps ~ N(0, noise).  Used for the 4-rank CPU configuration with
injected 50 ms sleeps.
"""
from __future__ import annotations

import torch
import torch.nn as nn


class HyperplaneRegressor(nn.Module):
    def __init__(self, dim: int = 4096):
        super().__init__()
        self.linear = nn.Linear(dim, 1, bias=False)
        nn.init.zeros_(self.linear.weight)

    def forward(self, x):
        return self.linear(x).squeeze(-1)


class HyperplaneData:
    """Seeded stream of (x, y) batches; every rank draws from its own sub-stream."""

    def __init__(self, dim: int = 4096, noise_std: float = 0.1, seed: int = 0, rank: int = 0):
        g = torch.Generator().manual_seed(seed)
        self.w_star = torch.randn(dim, generator=g)
        self.noise_std = noise_std
        self.dim = dim
        self.gen = torch.Generator().manual_seed(seed * 7919 + 1 + rank)

    def batch(self, n: int):
        x = torch.randn(n, self.dim, generator=self.gen)
        y = x @ self.w_star + self.noise_std * torch.randn(n, generator=self.gen)
        return x, y
