"""Video datasets in the layout of UCF101: clips of frames, class lists and train / test split files.

The reference loads UCF101 with PyAV (deep500/datasets/ucf101.py:18-109): every clip is decoded to RGB frames
of 240 x 320, optionally normalised with the data set's channel mean / std, the clips of a batch are
zero-padded ON THE LEFT to the longest one, then cut to ``[:max_length:skip_frames]``, scaled by 1/255 and put
channels-first, giving ``[batch, frames, 3, 240, 320]``.  No video decoder ships with this framework, so clips
are read from decoded arrays (one ``.npy`` of ``[frames, height, width, 3]`` uint8 per clip); everything
after decoding follows the reference.  ``write_synthetic_ucf101`` produces a small data set in that layout
(moving patterns whose direction and colour depend on the class) for tests and samples.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from .dataset import Dataset

UCF101_MEAN = (0.39607886, 0.37930175, 0.351559)
UCF101_STD = (0.28261574, 0.27613039, 0.28061599)


def read_split(root: str, split: str = "trainlist01.txt", class_index: str = "classInd.txt"):
    """``classInd.txt`` holds ``<1-based index> <class name>`` lines, a split file ``<class>/<clip> [index]``
    lines (deep500/datasets/ucf101.py:26-63).  Returns (paths, labels, class name -> index)."""
    classes: Dict[str, int] = {}
    with open(os.path.join(root, class_index)) as f:
        for line in f:
            if line.strip():
                idx, name = line.split()
                classes[name] = int(idx) - 1
    paths, labels = [], []
    with open(os.path.join(root, split)) as f:
        for line in f:
            if not line.strip():
                continue
            rel = line.split()[0]
            paths.append(os.path.join(root, os.path.splitext(rel)[0] + ".npy"))
            labels.append(classes[rel.split("/")[0]])
    return paths, np.asarray(labels, dtype=np.int64), classes


class VideoLoader:
    """Decoded clips -> a batch tensor, the reference's ``ucf101_loader`` after the decoder."""

    def __init__(self, normalize: bool = True, max_length: int = 1777, skip_frames: int = 10,
                 mean: Sequence[float] = UCF101_MEAN, std: Sequence[float] = UCF101_STD):
        self.normalize, self.max_length, self.skip_frames = normalize, max_length, skip_frames
        self.mean, self.std = np.asarray(mean, np.float32), np.asarray(std, np.float32)

    def _clip(self, path_or_array) -> np.ndarray:
        a = np.load(path_or_array) if isinstance(path_or_array, (str, os.PathLike)) else np.asarray(path_or_array)
        a = a.astype(np.float32)
        if self.normalize:
            a = (a - self.mean) / self.std
        return a

    def __call__(self, clips) -> np.ndarray:
        single = isinstance(clips, (str, os.PathLike)) or (isinstance(clips, np.ndarray) and clips.ndim == 4)
        data = [self._clip(c) for c in ([clips] if single else clips)]
        longest = max(x.shape[0] for x in data)
        data = [np.pad(x, ((longest - x.shape[0], 0), (0, 0), (0, 0), (0, 0))) for x in data]    # left padding
        batch = np.stack(data)[:, :self.max_length:self.skip_frames]
        batch = np.moveaxis(batch / 255.0, -1, -3)                                                # [B, T, 3, H, W]
        return batch[0] if single else batch


class VideoFolderDataset(Dataset):
    """Clips listed by a split file; a batch index returns ``{"x": [B, T, 3, H, W], "y": labels, "lengths"}``.
    ``lengths`` (frames per clip after sub-sampling) feeds ``BucketSampler``."""

    def __init__(self, root: str, split: str = "trainlist01.txt", loader: Optional[VideoLoader] = None,
                 data_node: str = "x", label_node: str = "y"):
        self.paths, self.labels, self.classes = read_split(root, split)
        self.loader = loader or VideoLoader()
        self.data_node, self.label_node = data_node, label_node
        raw = np.asarray([np.load(p, mmap_mode="r").shape[0] for p in self.paths], dtype=np.int64)
        self.lengths = np.asarray([len(range(0, min(int(n), self.loader.max_length), self.loader.skip_frames))
                                   for n in raw], dtype=np.int64)

    def __len__(self):
        return len(self.paths)

    def __getitem__(self, index):
        if isinstance(index, (int, np.integer)):
            return {self.data_node: self.loader(self.paths[index]), self.label_node: self.labels[index]}
        idx = list(range(*index.indices(len(self)))) if isinstance(index, slice) else list(index)
        return {self.data_node: self.loader([self.paths[i] for i in idx]), self.label_node: self.labels[idx],
                "lengths": self.lengths[idx]}


def write_synthetic_ucf101(root: str, classes: int = 4, clips_per_class: int = 6, frames: Tuple[int, int] = (20, 60),
                           size: Tuple[int, int] = (48, 64), seed: int = 0) -> str:
    """Write a tiny data set in the UCF101 layout: a bright bar sweeps across every frame, its direction, speed
    and colour are the class.  Returns ``root``."""
    rng = np.random.default_rng(seed)
    os.makedirs(root, exist_ok=True)
    names = ["Class%02d" % c for c in range(classes)]
    with open(os.path.join(root, "classInd.txt"), "w") as f:
        f.writelines("%d %s\n" % (c + 1, n) for c, n in enumerate(names))
    lines: List[Tuple[str, int]] = []
    h, w = size
    for c, name in enumerate(names):
        os.makedirs(os.path.join(root, name), exist_ok=True)
        for k in range(clips_per_class):
            t = int(rng.integers(frames[0], frames[1] + 1))
            clip = rng.integers(0, 40, size=(t, h, w, 3), dtype=np.uint8)
            for f_ in range(t):
                pos = (f_ * (c + 1)) % (w if c % 2 == 0 else h)
                if c % 2 == 0:
                    clip[f_, :, pos:pos + 4, c % 3] = 255
                else:
                    clip[f_, pos:pos + 4, :, c % 3] = 255
            rel = "%s/v_%s_g%02d_c01" % (name, name, k)
            np.save(os.path.join(root, rel + ".npy"), clip)
            lines.append((rel + ".avi", c + 1))
    order = rng.permutation(len(lines))
    n_test = max(classes, len(lines) // 4)
    with open(os.path.join(root, "testlist01.txt"), "w") as f:
        f.writelines("%s\n" % lines[i][0] for i in order[:n_test])
    with open(os.path.join(root, "trainlist01.txt"), "w") as f:
        f.writelines("%s %d\n" % lines[i] for i in order[n_test:])
    return root
