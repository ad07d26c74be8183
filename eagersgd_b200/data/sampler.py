"""Samplers: ordered, shuffled, length-bucketed, random choice, and their distributed forms.

Counterparts of deep500/lv2/sampler.py:14-301 (Sampler base with a seeded RandomState,
per-batch transformations and events; OrderedSampler, ShuffleSampler, BucketSampler,
ChoiceSampler) and deep500/lv3/distributed_sampler.py:10-114 (DistributedSampler,
PartitionedDataset, PartitionedDistributedSampler).
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence

import numpy as np

from .dataset import Dataset, collate_sequences


class Sampler:
    """Iterates over minibatches of a dataset.  Calling the sampler returns the next batch
    (a dict of arrays) or ``None`` at the end of the epoch; ``reset()`` starts a new epoch."""

    def __init__(self, dataset: Dataset, batch_size: int, seed: Optional[int] = None, drop_last_batch: bool = True,
                 events: Optional[Sequence] = None, transformations: Optional[Sequence[Callable]] = None):
        self.dataset, self.batch_size = dataset, int(batch_size)
        self.drop_last_batch = drop_last_batch
        self.events = list(events or [])
        self.transformations = list(transformations or [])
        self.seed = seed
        self.rng = np.random.RandomState(seed)
        self.batch_idx = 0
        self.epoch = 0

    def __len__(self) -> int:
        n = len(self.dataset)
        return n // self.batch_size if self.drop_last_batch else (n + self.batch_size - 1) // self.batch_size

    def __iter__(self):
        return self

    def __next__(self):
        b = self()
        if b is None:
            raise StopIteration
        return b

    def as_op(self):
        return self

    def add_input_transformation(self, fn: Callable):
        self.transformations.append(fn)

    def indices(self) -> Optional[np.ndarray]:
        """Sample indices of the next batch, or None when the epoch is over."""
        raise NotImplementedError

    def fetch(self, idx: np.ndarray) -> Dict[str, np.ndarray]:
        return self.dataset[idx]

    def __call__(self):
        for e in self.events:
            if hasattr(e, "before_sampling"):
                e.before_sampling(self, self.batch_size)
        idx = self.indices()
        if idx is None:
            return None
        batch = self.fetch(idx)
        for t in self.transformations:
            batch = t(batch)
        self.batch_idx += 1
        for e in self.events:
            if hasattr(e, "after_sampling"):
                e.after_sampling(self, self.batch_size)
        return batch

    def reset(self):
        self.batch_idx = 0
        for e in self.events:
            if hasattr(e, "on_sampler_reset"):
                e.on_sampler_reset(self)
        self.epoch += 1


class OrderedSampler(Sampler):
    def indices(self):
        lo = self.batch_idx * self.batch_size
        hi = lo + self.batch_size
        n = len(self.dataset)
        if lo >= n or (hi > n and self.drop_last_batch):
            return None
        return np.arange(lo, min(hi, n))


class ShuffleSampler(Sampler):
    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        self._perm = self.rng.permutation(len(self.dataset))

    def indices(self):
        lo = self.batch_idx * self.batch_size
        hi = lo + self.batch_size
        n = len(self.dataset)
        if lo >= n or (hi > n and self.drop_last_batch):
            return None
        return self._perm[lo:min(hi, n)]

    def reset(self):
        super().reset()
        self._perm = self.rng.permutation(len(self.dataset))


class ChoiceSampler(Sampler):
    """Batches drawn with replacement; an 'epoch' is len(dataset) // batch_size draws."""

    def indices(self):
        if self.batch_idx >= len(self):
            return None
        return self.rng.choice(len(self.dataset), self.batch_size, replace=True)


class BucketSampler(Sampler):
    """Variable-length sequences grouped into length buckets so that a batch pads little.

    ``lengths`` gives the length of every sample; ``num_buckets`` equal-width buckets up to
    ``max_length`` are formed (longer samples are truncated by ``fetch``).  Batches are drawn
    bucket by bucket in random order (deep500/lv2/sampler.py:159-241)."""

    def __init__(self, dataset: Dataset, batch_size: int, lengths: np.ndarray, num_buckets: int = 30,
                 max_length: Optional[int] = None, **kw):
        super().__init__(dataset, batch_size, **kw)
        self.lengths = np.asarray(lengths)
        self.max_length = int(max_length or self.lengths.max())
        edges = np.linspace(0, self.max_length, num_buckets + 1)
        which = np.clip(np.digitize(np.minimum(self.lengths, self.max_length), edges[1:-1]), 0, num_buckets - 1)
        self.buckets: List[np.ndarray] = [np.nonzero(which == b)[0] for b in range(num_buckets)]
        self._plan()

    def _plan(self):
        batches = []
        for members in self.buckets:
            if len(members) == 0:
                continue
            perm = self.rng.permutation(members)
            full = len(perm) // self.batch_size
            for i in range(full):
                batches.append(perm[i * self.batch_size:(i + 1) * self.batch_size])
            if not self.drop_last_batch and len(perm) % self.batch_size:
                batches.append(perm[full * self.batch_size:])
        order = self.rng.permutation(len(batches))
        self._batches = [batches[i] for i in order]

    def __len__(self):
        return len(self._batches)

    def indices(self):
        if self.batch_idx >= len(self._batches):
            return None
        return self._batches[self.batch_idx]

    def fetch(self, idx):
        items = [self.dataset[int(i)] for i in idx]
        seqs = [it[self.dataset.data_node][-self.max_length:] for it in items]
        return collate_sequences(seqs, np.asarray([it[self.dataset.label_node] for it in items]))

    def reset(self):
        super().reset()
        self._plan()


# ------------------------------------------------------------------------------ distributed
class DistributedSampler(Sampler):
    """Every rank holds the whole dataset and draws its own batches with a rank-specific seed;
    an epoch is 1/world of the data (deep500/lv3/distributed_sampler.py:10-40)."""

    def __init__(self, sampler: Sampler, rank=None, world: Optional[int] = None):
        """``DistributedSampler(sampler, rank, world)``, or ``DistributedSampler(sampler, group)`` with a process group
        (anything with ``rank`` and ``world`` attributes), as the reference passes its communicator; with neither, the
        rank and size of the running job."""
        if rank is not None and hasattr(rank, "rank") and hasattr(rank, "world"):
            rank, world = rank.rank, rank.world
        elif rank is None or world is None:
            import os
            rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
        self.__dict__.update(sampler.__dict__)
        self.inner, self.rank, self.world = sampler, int(rank), int(world)
        self.inner.rng = np.random.RandomState((sampler.seed or 0) * 9973 + rank)
        if hasattr(self.inner, "_perm"):
            self.inner._perm = self.inner.rng.permutation(len(sampler.dataset))

    def __len__(self):
        return len(self.inner) // self.world

    def __call__(self):
        if self.inner.batch_idx >= len(self):
            return None
        return self.inner()

    def reset(self):
        self.inner.reset()


class PartitionedDataset(Dataset):
    """A contiguous shard [lo, hi) of a dataset."""

    def __init__(self, dataset: Dataset, lo: int, hi: int):
        self.dataset, self.lo, self.hi = dataset, lo, hi
        for k in ("data_node", "label_node"):
            if hasattr(dataset, k):
                setattr(self, k, getattr(dataset, k))

    def __len__(self):
        return self.hi - self.lo

    def __getitem__(self, index):
        if isinstance(index, (int, np.integer)):
            return self.dataset[self.lo + int(index)]
        if isinstance(index, slice):
            index = np.arange(*index.indices(len(self)))
        return self.dataset[np.asarray(index) + self.lo]


def partition(dataset: Dataset, rank: int, world: int) -> PartitionedDataset:
    per = len(dataset) // world
    return PartitionedDataset(dataset, rank * per, (rank + 1) * per if rank < world - 1 else len(dataset))


class PartitionedDistributedSampler:
    """Each rank samples only its contiguous shard (distributed_sampler.py:100-108).  ``rank`` may be a process group."""

    def __new__(cls, sampler_cls, dataset=None, batch_size: Optional[int] = None, rank=None, world: Optional[int] = None, **kw):
        if isinstance(sampler_cls, Sampler):
            # the reference's form: PartitionedDistributedSampler(sampler, comm) narrows a ready sampler to the rank's shard
            s, comm = sampler_cls, dataset
            rank, world = (comm.rank, comm.world) if comm is not None else (0, 1)
            s.dataset = partition(s.dataset, rank, world)
            s.reset()                                       # a shuffled order is drawn again over the shard
            return s
        if hasattr(rank, "rank") and hasattr(rank, "world"):
            rank, world = rank.rank, rank.world
        return sampler_cls(partition(dataset, rank, world), batch_size, **kw)
