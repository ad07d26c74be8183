"""Batch transformations applied by samplers (deep500/frameworks/reference/augmentation.py:10-204):
ReplicateBatch, Crop (random / centre, with padding), Resize, Normalize, RandomFlip, Cutout, and the per-image
standardisation plus the CIFAR-10 recipe of the reference's main program.
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
    """Random or centre crop with optional constant padding; ``resize=True`` scales the crop back to the size the
    images had (nearest neighbour).  Arguments in the reference's order (augmentation.py:64-76)."""

    def __init__(self, crop_size: Sequence[int], resize: bool = False, random_crop: bool = False,
                 padding: Optional[Sequence[int]] = None, fill: float = 0.0, **kw):
        super().__init__(**kw)
        self.size, self.resize, self.random = tuple(crop_size), bool(resize), random_crop
        self.padding, self.fill = tuple(padding) if padding is not None else (0, 0), fill

    def apply(self, x):
        h0, w0 = x.shape[-2:]
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
        return Resize((h0, w0)).apply(out) if self.resize else out


class Resize(_Transform):
    """Nearest-neighbour resize to ``target_size`` (H, W)."""

    def __init__(self, target_size: Sequence[int], **kw):
        super().__init__(**kw)
        self.size = tuple(target_size)

    def apply(self, x):
        n, c, h, w = x.shape
        oh, ow = self.size
        ri = (np.arange(oh) * h / oh).astype(np.int64)
        ci = (np.arange(ow) * w / ow).astype(np.int64)
        return x[:, :, ri][:, :, :, ci]


class Normalize(_Transform):
    """(x - mean) / stddev per channel; a single number stands for every channel (augmentation.py:136-150)."""

    def __init__(self, mean=0.0, stddev=1.0, std=None, **kw):
        super().__init__(**kw)
        self.mean = np.asarray(mean, dtype=np.float32).reshape(1, -1, 1, 1)
        self.std = np.asarray(stddev if std is None else std, dtype=np.float32).reshape(1, -1, 1, 1)

    def apply(self, x):
        return (x - self.mean) / self.std


class RandomFlip(_Transform):
    """Mirror each sample along ``axis`` (default: the last, left-right) with probability ``p``
    (augmentation.py:152-165; there the test is inverted, so its probability is 1 - p: the same for the default)."""

    def __init__(self, axis: int = -1, p: float = 0.5, **kw):
        super().__init__(**kw)
        self.axis, self.prob = axis, p

    def apply(self, x):
        flip = self.rng.rand(x.shape[0]) < self.prob
        out = x.copy()
        axis = self.axis if self.axis < 0 else self.axis + 1          # axes are counted within one sample
        out[flip] = np.flip(out[flip], axis=axis)
        return out


class Cutout(_Transform):
    """Blank ``holes`` random squares of side ``length`` in every image (zero, or with ``random_fill`` uniform noise
    in [-0.5, 0.5)); arguments in the reference's order (augmentation.py:167-208)."""

    def __init__(self, holes: int = 1, length: int = 16, random_fill: bool = False, **kw):
        super().__init__(**kw)
        self.holes, self.length, self.random_fill = holes, length, random_fill

    def apply(self, x):
        out = x.copy()
        n, c, h, w = x.shape
        for i in range(n):
            for _ in range(self.holes):
                cy, cx = self.rng.randint(h), self.rng.randint(w)
                y0, y1 = max(0, cy - self.length // 2), min(h, cy + self.length // 2)
                x0, x1 = max(0, cx - self.length // 2), min(w, cx + self.length // 2)
                out[i, :, y0:y1, x0:x1] = (self.rng.rand(c, y1 - y0, x1 - x0) - 0.5) if self.random_fill else 0
        return out


class PerImageStandardization(_Transform):
    """(x - mean) / max(std, 1 / sqrt(elements)) over each image by itself — ``tf.image.per_image_standardization``,
    the last step of the reference's CIFAR-10 pipeline (official/resnet/cifar10_main.py:119-121)."""

    def apply(self, x):
        x = x.astype(np.float32, copy=False)
        flat = x.reshape(x.shape[0], -1)
        mean = flat.mean(axis=1)
        std = np.maximum(flat.std(axis=1), np.float32(1.0 / np.sqrt(flat.shape[1])))     # a float64 scalar would widen the batch
        shape = (-1,) + (1,) * (x.ndim - 1)
        return (x - mean.reshape(shape)) / std.reshape(shape)


def cifar10_transforms(is_training: bool, seed: Optional[int] = None, batchaug: int = 1, data_node: str = "x"):
    """The reference's CIFAR-10 input pipeline as a list of batch transformations: for training every image is padded
    by four pixels on each side, cropped back to 32 x 32 at a random offset and flipped with probability one half, then
    standardised by itself; for evaluation only the last step (official/resnet/cifar10_main.py:97-125).  With
    ``batchaug`` M every sample first appears M times, so that each copy gets its own crop and flip (:86-92)."""
    kw = dict(data_node=data_node)
    if not is_training:
        return [PerImageStandardization(**kw)]
    head = [ReplicateBatch(batchaug, **kw)] if batchaug and batchaug > 1 else []
    return head + [Crop((32, 32), random_crop=True, padding=(4, 4), seed=seed, **kw),
                   RandomFlip(seed=None if seed is None else seed + 1, **kw), PerImageStandardization(**kw)]
