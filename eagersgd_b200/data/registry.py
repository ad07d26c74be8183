"""Data sets by name: their shape, their loss, and a loader.

The reference's recipes and samples name a data set with a string and ask ``deep500.datasets`` for its shape
(``dataset_shape``: number of classes, then the shape of one sample), its loss (``dataset_loss``) and the two
``Dataset`` objects (``load_dataset(name, input_node, label_node, ...)``, which downloads what is missing:
deep500/datasets/__init__.py, deep500/recipe.py:63-107).  There is no network here, so a loader reads the files from
``path`` when one is given and otherwise hands out synthetic data of the data set's shape — a learnable task (every
class has a fixed random template, a sample is its class template plus noise), so that a recipe's accuracy bar still
means something.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional, Tuple

import numpy as np

from .dataset import Dataset, NumpyDataset, load_cifar10, load_cifar100, load_mnist, normalize_cifar

# name -> (classes, channels, height, width)
_SHAPES: Dict[str, Tuple] = {
    "mnist": (10, 1, 28, 28), "fashion_mnist": (10, 1, 28, 28), "cifar10": (10, 3, 32, 32), "cifar100": (100, 3, 32, 32),
    "imagenet": (1000, 3, 224, 224),
    "ucf101": (101, None, 3, 240, 320),            # clips of any number of frames (deep500/datasets/ucf101.py:18-19)
}


def dataset_shape(name: str) -> Tuple[int, ...]:
    """(classes, *shape of one sample)."""
    if name not in _SHAPES:
        raise KeyError("unknown data set %r (known: %s)" % (name, ", ".join(sorted(_SHAPES))))
    return _SHAPES[name]


def dataset_loss(name: str) -> Callable:
    """The loss a model is trained with on this data set: softmax cross-entropy for all of the above."""
    dataset_shape(name)
    from ..train.executor import classification_loss
    return classification_loss


def synthetic_task(classes: int, shape: Tuple[int, ...], samples: int, input_node: str = "x", label_node: str = "y",
                   seed: int = 0, noise: float = 1.0, templates_seed: int = 12345) -> NumpyDataset:
    """``samples`` draws of a task a network can learn: half a fixed per-class template plus unit Gaussian noise."""
    templates = np.random.RandomState(templates_seed).randn(classes, *shape).astype(np.float32)
    rng = np.random.RandomState(seed)
    y = rng.randint(0, classes, size=samples).astype(np.int64)
    x = 0.5 * templates[y] + noise * rng.randn(samples, *shape).astype(np.float32)
    return NumpyDataset(x, input_node, y, label_node)


def _renamed(ds: Dataset, input_node: str, label_node: str) -> Dataset:
    if getattr(ds, "data_node", input_node) == input_node and getattr(ds, "label_node", label_node) == label_node:
        return ds
    both = ds[:]
    return NumpyDataset(both[ds.data_node], input_node, both[ds.label_node], label_node)


def load_dataset(name: str, input_node: str = "x", label_node: str = "y", path: Optional[str] = None,
                 synthetic_samples: int = 512, seed: int = 0, noise: float = 1.0, normalize: bool = True
                 ) -> Tuple[Dataset, Dataset]:
    """(training set, validation set) with the given node names.  ``path``: where the files are (CIFAR-10 batch files,
    CIFAR-100 ``train.bin`` / ``test.bin``, MNIST / Fashion-MNIST idx files, ImageNet class folders; CIFAR images are
    normalised by the data set's channel statistics unless ``normalize=False``); without it, synthetic data of the right shape
    (``synthetic_samples`` training samples with Gaussian noise of standard deviation ``noise`` around the templates)."""
    classes, *shape = dataset_shape(name)
    if name == "ucf101":
        if path is None:
            raise FileNotFoundError("ucf101 needs path= (frame folders and the trainlist / testlist split files)")
        from .video import VideoFolderDataset
        return (VideoFolderDataset(path, "trainlist01.txt", data_node=input_node, label_node=label_node),
                VideoFolderDataset(path, "testlist01.txt", data_node=input_node, label_node=label_node))
    if path is None:
        return (synthetic_task(classes, tuple(shape), synthetic_samples, input_node, label_node, seed=seed + 1, noise=noise),
                synthetic_task(classes, tuple(shape), max(synthetic_samples // 4, 32), input_node, label_node, seed=seed + 2,
                               noise=noise))
    if name in ("cifar10", "cifar100"):
        train, test = (load_cifar10 if name == "cifar10" else load_cifar100)(path)
        if normalize:                           # the reference's loaders normalise by the channel statistics by default
            train, test = normalize_cifar(train, name), normalize_cifar(test, name)
    elif name in ("mnist", "fashion_mnist"):
        train, test = load_mnist(path)
    elif name == "imagenet":
        from .imagenet import ImageNetFolder
        train, test = ImageNetFolder(path, "train", seed=seed), ImageNetFolder(path, "val", seed=seed)
        if (input_node, label_node) != ("x", "y"):
            raise ValueError("ImageNet is decoded on access and keeps the node names 'x' and 'y'")
        return train, test
    else:
        raise FileNotFoundError("no reader for %s files; leave the path out for synthetic data of its shape" % name)
    return _renamed(train, input_node, label_node), _renamed(test, input_node, label_node)
