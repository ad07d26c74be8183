"""Optimizers: eager-SGD wrappers and companions."""
from .eager import (EagerOptimizer, SoloAllreduceOptimizer, MajorityAllreduceOptimizer,  # noqa: F401
                    SyncAllreduceOptimizer)
