"""Datasets, samplers and augmentation."""
from .dataset import (Dataset, NumpyDataset, FileListDataset, SyntheticImageDataset,  # noqa: F401
                      SyntheticSequenceDataset, collate_sequences, load_cifar10, load_mnist)
from .sampler import (Sampler, OrderedSampler, ShuffleSampler, ChoiceSampler, BucketSampler,  # noqa: F401
                      DistributedSampler, PartitionedDataset, PartitionedDistributedSampler, partition)
from .augmentation import ReplicateBatch, Crop, Resize, Normalize, RandomFlip, Cutout  # noqa: F401
