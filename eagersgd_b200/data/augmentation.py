"""Batch transformations applied by samplers (deep500/frameworks/reference/augmentation.py:10-204):
ReplicateBatch, Crop (random / centre, with padding), Resize, Normalize, RandomFlip, Cutout.
Batches are dicts of numpy arrays with images in NCHW under ``data_node``."""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import numpy as np


class _Transform:
    def __init__(self, data_node: str = "x", seed: Optional[int] = None):
        self.node = data_node
        self.rng = np.random.RandomState(seed)

    def __call__(self, batch: Dict[str, np.ndarray]) -> Dict[str, np.ndarray]:
        out = dict(batch)
        out[self.node] = self.apply(batch[self.node])
        return out

    def apply(self, x: np.ndarray) -> np.ndarray:
        raise NotImplementedError


class ReplicateBatch(_Transform):
    """Repeat every sample ``duplicates`` times (batch augmentation)."""

    def __init__(self, duplicates: int, **kw):
        super().__init__(**kw)
        self.duplicates = duplicates

    def __call__(self, batch):
        return {k: np.repeat(v, self.duplicates, axis=0) for k, v in batch.items()}


class Crop(_Transform):
    def __init__(self, crop_size: Sequence[int], random_crop: bool = False, padding: Sequence[int] = (0, 0),
                 fill: float = 0.0, **kw):
        super().__init__(**kw)
        self.size, self.random, self.padding, self.fill = tuple(crop_size), random_crop, tuple(padding), fill

    def apply(self, x):
        ph, pw = self.padding
        if ph or pw:
            x = np.pad(x, ((0, 0), (0, 0), (ph, ph), (pw, pw)), constant_values=self.fill)
        n, c, h, w = x.shape
        ch, cw = self.size
        out = np.empty((n, c, ch, cw), dtype=x.dtype)
        for i in range(n):
            if self.random:
                t, l = self.rng.randint(0, h - ch + 1), self.rng.randint(0, w - cw + 1)
            else:
                t, l = (h - ch) // 2, (w - cw) // 2
            out[i] = x[i, :, t:t + ch, l:l + cw]
        return out


class Resize(_Transform):
    """Nearest-neighbour resize to ``size`` (H, W)."""

    def __init__(self, size: Sequence[int], **kw):
        super().__init__(**kw)
        self.size = tuple(size)

    def apply(self, x):
        n, c, h, w = x.shape
        oh, ow = self.size
        ri = (np.arange(oh) * h / oh).astype(np.int64)
        ci = (np.arange(ow) * w / ow).astype(np.int64)
        return x[:, :, ri][:, :, :, ci]


class Normalize(_Transform):
    def __init__(self, mean: Sequence[float], std: Sequence[float], **kw):
        super().__init__(**kw)
        self.mean = np.asarray(mean, dtype=np.float32).reshape(1, -1, 1, 1)
        self.std = np.asarray(std, dtype=np.float32).reshape(1, -1, 1, 1)

    def apply(self, x):
        return (x - self.mean) / self.std


class RandomFlip(_Transform):
    def __init__(self, prob: float = 0.5, **kw):
        super().__init__(**kw)
        self.prob = prob

    def apply(self, x):
        flip = self.rng.rand(x.shape[0]) < self.prob
        out = x.copy()
        out[flip] = out[flip, :, :, ::-1]
        return out


class Cutout(_Transform):
    """Zero one random square of side ``length`` per image."""

    def __init__(self, length: int, **kw):
        super().__init__(**kw)
        self.length = length

    def apply(self, x):
        out = x.copy()
        n, _, h, w = x.shape
        for i in range(n):
            cy, cx = self.rng.randint(h), self.rng.randint(w)
            y0, y1 = max(0, cy - self.length // 2), min(h, cy + self.length // 2)
            x0, x1 = max(0, cx - self.length // 2), min(w, cx + self.length // 2)
            out[i, :, y0:y1, x0:x1] = 0
        return out
