"""Datasets, samplers and augmentation."""
from .dataset import (Dataset, NumpyDataset, FileListDataset, SyntheticImageDataset,  # noqa: F401
                      SyntheticSequenceDataset, collate_sequences, load_cifar10, load_mnist)
from .sampler import (Sampler, OrderedSampler, ShuffleSampler, ChoiceSampler, BucketSampler,  # noqa: F401
                      DistributedSampler, PartitionedDataset, PartitionedDistributedSampler, partition)
from .augmentation import (ReplicateBatch, Crop, Resize, Normalize, RandomFlip, Cutout, PerImageStandardization,  # noqa: F401
                           cifar10_transforms)
from .video import VideoLoader, VideoFolderDataset, read_split, write_synthetic_ucf101, UCF101_MEAN, UCF101_STD  # noqa: F401
from .imagenet import (ImageNetFolder, ShardedImageDataset, SyntheticImageNet, build_shards, preprocess_image,  # noqa: F401
                       random_crop_box, decode_image, write_synthetic_imagenet, CHANNEL_MEANS)
from .registry import dataset_shape, dataset_loss, load_dataset, synthetic_task  # noqa: F401
from .dataset import load_cifar100, normalize_cifar, cifar_learning_rate, CIFAR_MEAN, CIFAR_STD  # noqa: F401
