"""eagersgd_b200 — eager-SGD (partial-collective, stale-synchronous data-parallel
training) designed for NVIDIA B200: sm_100a kernels, NVLink 5 / NVSwitch peer
memory, one process per GPU.

Layout
------
parallel/  process group, partial allreduce (NVLink kernels, CPU shared-memory backend)
optim/     Solo/Majority/Sync optimizer wrappers, fused SGD, LARS, parity optimizers
ops/       hand-written kernels behind autograd functions, op JIT + validation
models/    ResNet (CIFAR / ImageNet), LSTM classifier, hyperplane regressor, MNIST nets
data/      synthetic datasets, samplers, augmentation
train/     trainer, events, metrics, flags, imbalance injectors, command-line mains
ckpt/      checkpoints in the tf-models ResNet variable layout, rank-0 re-sync
ref/       CPU oracles (numpy / C++) for every kernel
"""
__version__ = "0.2.0"

from .parallel.group import Group, init, finalize, rank, world_size  # noqa: F401
from .parallel.partial_allreduce import PartialAllreduce  # noqa: F401
from .optim.eager import (EagerOptimizer, SoloAllreduceOptimizer, MajorityAllreduceOptimizer,  # noqa: F401
                          SyncAllreduceOptimizer)

_SUBPACKAGES = ("train", "data", "models", "optim", "ops", "graph", "ckpt", "utils", "recipes", "parallel", "ref")


def __getattr__(name):
    """``import eagersgd_b200 as es; es.train.prepare_model(...)``: sub-packages are imported when first asked for."""
    if name in _SUBPACKAGES:
        import importlib
        return importlib.import_module("." + name, __name__)
    raise AttributeError("module %r has no attribute %r" % (__name__, name))
