"""Launch helper (re-exec a script as N ranks), device descriptors, measured peaks."""
from .launch import fork, rank_env, free_port  # noqa: F401
from .device import CPUDevice, GPUDevice, DeviceType, describe, measured_peaks  # noqa: F401
from .nvtx import nvtx_range, nvtx_enabled  # noqa: F401
from . import download  # noqa: F401
