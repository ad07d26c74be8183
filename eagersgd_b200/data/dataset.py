"""Datasets: in-memory arrays, file lists and the synthetic sets the benchmarks use.

Counterparts of the reference's ``Dataset`` / ``NumpyDataset`` / ``FileListDataset``
(deep500/lv2/dataset.py:6-134) and of its synthetic ImageNet input
(deep500/datasets/imagenet.py:84-107, official/resnet/resnet_run_loop_solo_imagenet_300.py:134-158).
There is no network here, so the real-data loaders take local paths only.
"""
from __future__ import annotations

import os
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np


class Dataset:
    """Indexable collection of samples; ``dataset[i]`` returns a dict name -> array."""

    def __len__(self) -> int:
        raise NotImplementedError

    def __getitem__(self, index):
        raise NotImplementedError

    def add_label_to_sample(self, label_node: str):
        self.label_node = label_node


class NumpyDataset(Dataset):
    def __init__(self, data: np.ndarray, data_node: str = "x", labels: Optional[np.ndarray] = None,
                 label_node: str = "y"):
        self.data, self.labels = data, labels
        self.data_node, self.label_node = data_node, label_node

    def __len__(self):
        return len(self.data)

    def __getitem__(self, index):
        out = {self.data_node: self.data[index]}
        if self.labels is not None:
            out[self.label_node] = self.labels[index]
        return out


class FileListDataset(Dataset):
    """Files decoded on access by ``file_to_array`` (a callable path -> ndarray)."""

    def __init__(self, filenames: Sequence[str], data_node: str, labels: np.ndarray, label_node: str,
                 file_to_array: Callable[[str], np.ndarray]):
        self.filenames, self.labels = list(filenames), labels
        self.data_node, self.label_node = data_node, label_node
        self.file_to_array = file_to_array

    def __len__(self):
        return len(self.filenames)

    def __getitem__(self, index):
        if isinstance(index, (slice, list, np.ndarray)):
            idx = range(*index.indices(len(self))) if isinstance(index, slice) else index
            data = np.stack([self.file_to_array(self.filenames[i]) for i in idx])
            return {self.data_node: data, self.label_node: self.labels[list(idx)]}
        return {self.data_node: self.file_to_array(self.filenames[index]), self.label_node: self.labels[index]}


class SyntheticImageDataset(Dataset):
    """N(0,1) images with uniform labels, generated on demand from (seed, index)."""

    def __init__(self, length: int, shape: Tuple[int, int, int] = (3, 224, 224), classes: int = 1000, seed: int = 0,
                 dtype=np.float32):
        self.length, self.shape, self.classes, self.seed, self.dtype = length, shape, classes, seed, dtype
        self.data_node, self.label_node = "x", "y"

    def __len__(self):
        return self.length

    def _one(self, i: int):
        rng = np.random.default_rng(self.seed * 1000003 + int(i))
        return rng.standard_normal(self.shape, dtype=np.float32).astype(self.dtype), int(rng.integers(self.classes))

    def __getitem__(self, index):
        if isinstance(index, (int, np.integer)):
            x, y = self._one(index)
            return {"x": x, "y": np.int64(y)}
        idx = range(*index.indices(self.length)) if isinstance(index, slice) else index
        xs, ys = zip(*[self._one(i) for i in idx])
        return {"x": np.stack(xs), "y": np.asarray(ys, dtype=np.int64)}


class SyntheticSequenceDataset(Dataset):
    """Variable-length feature sequences: lengths from a clipped log-normal over
    [min_len, max_len] frames, features N(0,1) of ``feature_dim``, uniform labels over
    ``classes`` — the video-classification workload whose length spread is the natural
    load imbalance (deep500/datasets/ucf101.py:69-109 loads real frames the same way)."""

    def __init__(self, length: int, feature_dim: int = 2048, classes: int = 101, min_len: int = 30,
                 max_len: int = 1800, mu: float = 5.2, sigma: float = 0.6, seed: int = 0):
        rng = np.random.default_rng(seed)
        self.lengths = np.clip(rng.lognormal(mu, sigma, size=length), min_len, max_len).astype(np.int64)
        self.labels = rng.integers(classes, size=length).astype(np.int64)
        self.feature_dim, self.classes, self.seed = feature_dim, classes, seed
        self.data_node, self.label_node = "x", "y"

    def __len__(self):
        return len(self.lengths)

    def sequence(self, i: int) -> np.ndarray:
        rng = np.random.default_rng(self.seed * 7919 + 13 + int(i))
        return rng.standard_normal((int(self.lengths[i]), self.feature_dim), dtype=np.float32)

    def __getitem__(self, index):
        if isinstance(index, (int, np.integer)):
            return {"x": self.sequence(index), "y": self.labels[index]}
        idx = list(range(*index.indices(len(self)))) if isinstance(index, slice) else list(index)
        return collate_sequences([self.sequence(i) for i in idx], self.labels[idx])


def collate_sequences(seqs: List[np.ndarray], labels: np.ndarray) -> Dict[str, np.ndarray]:
    """Left-zero-pad to the longest sequence of the batch (the reference pads on the left too,
    deep500/datasets/ucf101.py:92-109) and return the true lengths."""
    t = max(len(s) for s in seqs)
    out = np.zeros((len(seqs), t) + tuple(seqs[0].shape[1:]), dtype=seqs[0].dtype)   # frames of any rank
    for i, s in enumerate(seqs):
        out[i, t - len(s):] = s
    return {"x": out, "y": np.asarray(labels), "lengths": np.asarray([len(s) for s in seqs], dtype=np.int64)}


def load_cifar10(path: str):
    """CIFAR-10 from a local directory (no download): returns train / test ``NumpyDataset``s of float32 images in
    [0, 1], NCHW, with int64 labels.  Both published forms are read: the binary one the reference's main program uses
    (``cifar-10-batches-bin/data_batch_{1..5}.bin`` and ``test_batch.bin``, records of one label byte followed by
    3 x 32 x 32 pixel bytes, channel-major: official/resnet/cifar10_main.py:33-95) and the pickled "python" one
    (``cifar-10-batches-py/data_batch_{1..5}``, ``test_batch``).  ``path`` is the directory with the batch files or
    the one that holds the ``cifar-10-batches-*`` folder."""
    import pickle

    for sub in ("", "cifar-10-batches-bin", "cifar-10-batches-py"):
        d = os.path.join(path, sub)
        if os.path.exists(os.path.join(d, "data_batch_1.bin")) or os.path.exists(os.path.join(d, "data_batch_1")):
            path = d
            break
    else:
        raise FileNotFoundError("no CIFAR-10 batch files (data_batch_1.bin or data_batch_1) under %s" % path)

    def _read_bin(fn):
        raw = np.fromfile(os.path.join(path, fn), dtype=np.uint8)
        if raw.size % 3073:
            raise ValueError("%s is not a sequence of 3073-byte CIFAR-10 records" % fn)
        rec = raw.reshape(-1, 3073)
        return rec[:, 1:].reshape(-1, 3, 32, 32).astype(np.float32) / 255.0, rec[:, 0].astype(np.int64)

    def _read_py(fn):
        with open(os.path.join(path, fn), "rb") as f:
            d = pickle.load(f, encoding="bytes")
        return d[b"data"].reshape(-1, 3, 32, 32).astype(np.float32) / 255.0, np.asarray(d[b"labels"], dtype=np.int64)

    binary = os.path.exists(os.path.join(path, "data_batch_1.bin"))
    read, ext = (_read_bin, ".bin") if binary else (_read_py, "")
    xs, ys = zip(*[read("data_batch_%d%s" % (i, ext)) for i in range(1, 6)])
    tx, ty = read("test_batch" + ext)
    return NumpyDataset(np.concatenate(xs), "x", np.concatenate(ys), "y"), NumpyDataset(tx, "x", ty, "y")


# channel statistics and the fast learning-rate schedule the reference ships with its CIFAR loaders
# (deep500/datasets/cifar.py:58-78)
CIFAR_MEAN = {"cifar10": (0.4914, 0.4822, 0.4465), "cifar100": (0.5071, 0.4867, 0.4408)}
CIFAR_STD = {"cifar10": (0.2023, 0.1994, 0.2010), "cifar100": (0.2675, 0.2565, 0.2761)}


def cifar_learning_rate(epoch: int, init: float = 0.1) -> float:
    """init x 0.2 ^ k with k = 1, 2, 3 after epochs 60, 120, 160."""
    return init * 0.2 ** sum(epoch > e for e in (60, 120, 160))


def normalize_cifar(ds: "NumpyDataset", name: str = "cifar10") -> "NumpyDataset":
    """Subtract the data set's channel means and divide by its channel deviations (images in [0, 1])."""
    mean = np.asarray(CIFAR_MEAN[name], dtype=np.float32).reshape(1, 3, 1, 1)
    std = np.asarray(CIFAR_STD[name], dtype=np.float32).reshape(1, 3, 1, 1)
    both = ds[:]
    return NumpyDataset((both[ds.data_node] - mean) / std, ds.data_node, both[ds.label_node], ds.label_node)


def load_cifar100(path: str):
    """CIFAR-100 in its binary form (``cifar-100-binary/train.bin``, ``test.bin``: records of a coarse-label byte, a
    fine-label byte and 3 x 32 x 32 pixel bytes): train / test ``NumpyDataset``s with the fine labels
    (deep500/datasets/cifar.py:80-116 reads the same files)."""
    for sub in ("", "cifar-100-binary"):
        d = os.path.join(path, sub)
        if os.path.exists(os.path.join(d, "train.bin")):
            path = d
            break
    else:
        raise FileNotFoundError("no CIFAR-100 files (train.bin, test.bin) under %s" % path)

    def _read(fn):
        raw = np.fromfile(os.path.join(path, fn), dtype=np.uint8)
        if raw.size % 3074:
            raise ValueError("%s is not a sequence of 3074-byte CIFAR-100 records" % fn)
        rec = raw.reshape(-1, 3074)
        return rec[:, 2:].reshape(-1, 3, 32, 32).astype(np.float32) / 255.0, rec[:, 1].astype(np.int64)

    (x, y), (tx, ty) = _read("train.bin"), _read("test.bin")
    return NumpyDataset(x, "x", y, "y"), NumpyDataset(tx, "x", ty, "y")


def load_mnist(path: str):
    """MNIST idx files from a local directory."""
    import gzip
    import struct

    def _idx(fn):
        op = gzip.open if fn.endswith(".gz") else open
        with op(os.path.join(path, fn), "rb") as f:
            magic, = struct.unpack(">I", f.read(4))
            dims = struct.unpack(">" + "I" * (magic & 0xFF), f.read(4 * (magic & 0xFF)))
            return np.frombuffer(f.read(), dtype=np.uint8).reshape(dims)

    def _find(stem):
        for ext in ("", ".gz"):
            if os.path.exists(os.path.join(path, stem + ext)):
                return stem + ext
        raise FileNotFoundError(stem)

    tr_x = _idx(_find("train-images-idx3-ubyte")).astype(np.float32)[:, None] / 255.0
    tr_y = _idx(_find("train-labels-idx1-ubyte")).astype(np.int64)
    te_x = _idx(_find("t10k-images-idx3-ubyte")).astype(np.float32)[:, None] / 255.0
    te_y = _idx(_find("t10k-labels-idx1-ubyte")).astype(np.int64)
    return NumpyDataset(tr_x, "x", tr_y, "y"), NumpyDataset(te_x, "x", te_y, "y")
