"""ImageNet from disk: the folder layout, packed shards, and the reference's pre-processing.

* ``ImageNetFolder``: ``<root>/<split>/<wnid>/*.JPEG`` (one directory per class), decoded with PIL.
* ``build_shards`` / ``ShardedImageDataset``: the encoded files of a split packed into a few large shard files
  with labels (what the reference's TFRecord builder and reader do: official/resnet/build_imagenet_data.py,
  imagenet_main_eagersgd.py:60-160 ``parse_record``), so that a training job opens tens of files, not a million.
* ``preprocess_image``: official/resnet/imagenet_preprocessing.py — training: a random crop covering 5 %..100 %
  of the image with aspect ratio in [3/4, 4/3] (falling back to the whole image), random horizontal flip,
  resize to 224 x 224; evaluation: aspect-preserving resize to a shorter side of 256 and the central 224 x 224
  crop; both subtract the channel means (123.68, 116.78, 103.94) and leave the 0..255 scale.
* ``SyntheticImageNet``: the reference's synthetic input (imagenet.py:84-107, run loop :134-158): constant random
  images of the right shape and labels, for input-pipeline-free benchmarking.

Labels are 0-based over the sorted class directories; ``label_offset=1`` reproduces the reference's 1001-class
convention with a background class 0.
"""
from __future__ import annotations

import io
import os
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from .dataset import Dataset

CHANNEL_MEANS = (123.68, 116.78, 103.94)
DEFAULT_SIZE = 224
RESIZE_MIN = 256
_EXT = (".jpeg", ".jpg", ".png", ".bmp", ".ppm")


def _pil():
    from PIL import Image
    return Image


def decode_image(data) -> np.ndarray:
    """Encoded bytes or a path -> uint8 [H, W, 3]."""
    Image = _pil()
    img = Image.open(io.BytesIO(data) if isinstance(data, (bytes, bytearray, memoryview)) else data)
    return np.asarray(img.convert("RGB"))


def _resize(img: np.ndarray, h: int, w: int) -> np.ndarray:
    Image = _pil()
    return np.asarray(Image.fromarray(img).resize((w, h), Image.BILINEAR))


def random_crop_box(h: int, w: int, rng: np.random.Generator, area=(0.05, 1.0), ratio=(0.75, 4.0 / 3.0),
                    attempts: int = 100) -> Tuple[int, int, int, int]:
    """(top, left, height, width) of a crop with the given relative area and aspect ratio; the whole image if no
    attempt fits (tf.image.sample_distorted_bounding_box with the whole image as the only box)."""
    for _ in range(attempts):
        a = rng.uniform(*area) * h * w
        r = rng.uniform(*ratio)
        cw, ch = int(round(np.sqrt(a * r))), int(round(np.sqrt(a / r)))
        if 0 < cw <= w and 0 < ch <= h:
            return int(rng.integers(0, h - ch + 1)), int(rng.integers(0, w - cw + 1)), ch, cw
    return 0, 0, h, w


def preprocess_image(img: np.ndarray, is_training: bool, rng: Optional[np.random.Generator] = None,
                     size: int = DEFAULT_SIZE, means: Sequence[float] = CHANNEL_MEANS) -> np.ndarray:
    """uint8 [H, W, 3] -> float32 [3, size, size], mean-subtracted, 0..255 scale."""
    h, w = img.shape[:2]
    if is_training:
        rng = rng or np.random.default_rng()
        t, l, ch, cw = random_crop_box(h, w, rng)
        img = img[t:t + ch, l:l + cw]
        if rng.random() < 0.5:
            img = img[:, ::-1]
        img = _resize(np.ascontiguousarray(img), size, size)
    else:
        scale = RESIZE_MIN / min(h, w)
        nh, nw = max(int(round(h * scale)), size), max(int(round(w * scale)), size)
        img = _resize(img, nh, nw)
        t, l = (nh - size) // 2, (nw - size) // 2
        img = img[t:t + size, l:l + size]
    out = img.astype(np.float32) - np.asarray(means, np.float32)
    return np.ascontiguousarray(np.moveaxis(out, -1, 0))


def list_folder(root: str, split: str) -> Tuple[List[str], np.ndarray, List[str]]:
    base = os.path.join(root, split)
    classes = sorted(d for d in os.listdir(base) if os.path.isdir(os.path.join(base, d)))
    files, labels = [], []
    for c, name in enumerate(classes):
        for fn in sorted(os.listdir(os.path.join(base, name))):
            if fn.lower().endswith(_EXT):
                files.append(os.path.join(base, name, fn))
                labels.append(c)
    return files, np.asarray(labels, dtype=np.int64), classes


class _ImageDataset(Dataset):
    data_node, label_node = "x", "y"

    num_parallel_calls = 1      # threads that decode and pre-process the images of one batch
    batchaug = 1                # training batches hold every sample this many times, each copy cropped and flipped by itself
                                # (the reference tiles the encoded image before its pre-processing: imagenet_main_eagersgd.py:149-154)

    def _init_common(self, is_training, size, seed, label_offset):
        self.is_training, self.size, self.label_offset = is_training, size, label_offset
        self.rng = np.random.default_rng(seed)
        self._pool = None

    def _raw(self, i: int):
        raise NotImplementedError

    def __getitem__(self, index):
        if isinstance(index, (int, np.integer)):
            return {"x": preprocess_image(decode_image(self._raw(int(index))), self.is_training, self.rng, self.size),
                    "y": self.labels[index] + self.label_offset}
        idx = list(range(*index.indices(len(self)))) if isinstance(index, slice) else list(index)
        if self.is_training and self.batchaug > 1:
            idx = [i for i in idx for _ in range(self.batchaug)]
        if self.num_parallel_calls > 1:       # like dataset.map(parse_record, num_parallel_calls=n) in the reference
            if self._pool is None:
                from concurrent.futures import ThreadPoolExecutor
                self._pool = ThreadPoolExecutor(self.num_parallel_calls)
            seeds = self.rng.integers(1 << 62, size=len(idx))
            x = np.stack(list(self._pool.map(
                lambda a: preprocess_image(decode_image(self._raw(int(a[0]))), self.is_training,
                                           np.random.default_rng(int(a[1])), self.size), zip(idx, seeds))))
        else:
            x = np.stack([preprocess_image(decode_image(self._raw(int(i))), self.is_training, self.rng, self.size)
                          for i in idx])
        return {"x": x, "y": self.labels[idx] + self.label_offset}


class ImageNetFolder(_ImageDataset):
    def __init__(self, root: str, split: str = "train", is_training: Optional[bool] = None, size: int = DEFAULT_SIZE,
                 seed: int = 0, label_offset: int = 0):
        self.files, self.labels, self.classes = list_folder(root, split)
        self._init_common(split == "train" if is_training is None else is_training, size, seed, label_offset)

    def __len__(self):
        return len(self.files)

    def _raw(self, i):
        return self.files[i]


def build_shards(root: str, split: str, out_dir: str, shard_size: int = 1024) -> List[str]:
    """Pack the encoded image files of ``<root>/<split>`` into ``<out_dir>/<split>-00000-of-0000N.npz`` shards
    (bytes, offsets, labels, class names) in a seeded shuffled order, as the reference's record builder does."""
    files, labels, classes = list_folder(root, split)
    order = np.random.default_rng(12345).permutation(len(files))
    os.makedirs(out_dir, exist_ok=True)
    n_shards = max((len(files) + shard_size - 1) // shard_size, 1)
    out = []
    for s in range(n_shards):
        part = order[s * shard_size:(s + 1) * shard_size]
        blobs = [open(files[i], "rb").read() for i in part]
        offsets = np.cumsum([0] + [len(b) for b in blobs]).astype(np.int64)
        path = os.path.join(out_dir, "%s-%05d-of-%05d.npz" % (split, s, n_shards))
        np.savez(path, data=np.frombuffer(b"".join(blobs), dtype=np.uint8), offsets=offsets,
                 labels=labels[part], classes=np.asarray(classes))
        out.append(path)
    return out


class ShardedImageDataset(_ImageDataset):
    """Reads what ``build_shards`` wrote; shards are opened lazily and kept memory-mapped per process."""

    def __init__(self, shard_dir: str, split: str = "train", is_training: Optional[bool] = None,
                 size: int = DEFAULT_SIZE, seed: int = 0, label_offset: int = 0):
        self.paths = sorted(os.path.join(shard_dir, f) for f in os.listdir(shard_dir)
                            if f.startswith(split + "-") and f.endswith(".npz"))
        if not self.paths:
            raise FileNotFoundError("no %s-*.npz shards in %s" % (split, shard_dir))
        self._shards: Dict[int, dict] = {}
        counts, labels = [], []
        for p in self.paths:
            with np.load(p) as z:
                counts.append(len(z["labels"]))
                labels.append(z["labels"])
                self.classes = [str(c) for c in z["classes"]]
        self.starts = np.cumsum([0] + counts)
        self.labels = np.concatenate(labels).astype(np.int64)
        self._init_common(split == "train" if is_training is None else is_training, size, seed, label_offset)

    def __len__(self):
        return int(self.starts[-1])

    def _raw(self, i):
        s = int(np.searchsorted(self.starts, i, side="right") - 1)
        if s not in self._shards:
            z = np.load(self.paths[s])
            self._shards[s] = {"data": z["data"], "offsets": z["offsets"]}
        sh = self._shards[s]
        j = i - int(self.starts[s])
        return sh["data"][sh["offsets"][j]:sh["offsets"][j + 1]].tobytes()


class SyntheticImageNet(Dataset):
    """One fixed random batch repeated: measures training without an input pipeline."""
    data_node, label_node = "x", "y"

    def __init__(self, length: int = 1281167, size: int = DEFAULT_SIZE, classes: int = 1000, seed: int = 0):
        rng = np.random.default_rng(seed)
        self.length, self.classes = length, classes
        self._img = (rng.standard_normal((3, size, size)) * 60.0).astype(np.float32)
        self._label = int(rng.integers(classes))

    def __len__(self):
        return self.length

    def __getitem__(self, index):
        if isinstance(index, (int, np.integer)):
            return {"x": self._img, "y": np.int64(self._label)}
        n = len(range(*index.indices(self.length))) if isinstance(index, slice) else len(index)
        return {"x": np.broadcast_to(self._img, (n,) + self._img.shape), "y": np.full(n, self._label, np.int64)}


def write_synthetic_imagenet(root: str, classes: int = 3, per_class: int = 4, seed: int = 0) -> str:
    """A few small JPEG files in the ImageNet folder layout (train / val), for tests and samples."""
    Image = _pil()
    rng = np.random.default_rng(seed)
    for split, n in (("train", per_class), ("val", max(per_class // 2, 1))):
        for c in range(classes):
            d = os.path.join(root, split, "n%08d" % (1000 + c))
            os.makedirs(d, exist_ok=True)
            for k in range(n):
                h, w = int(rng.integers(40, 90)), int(rng.integers(40, 90))
                img = rng.integers(0, 255, size=(h, w, 3), dtype=np.uint8)
                img[..., c % 3] = 255 - img[..., c % 3] // 4        # the class tints the image
                Image.fromarray(img).save(os.path.join(d, "img_%d.JPEG" % k), quality=90)
    return root
