"""Device descriptors and the machine's measured peaks.

``CPUDevice`` / ``GPUDevice`` mirror the reference's executor device arguments (deep500/utils/device.py);
``describe()`` reports what the kernels of this package are written for and what the machine measured.
"""
from __future__ import annotations

import json
import os
from typing import Optional

import torch

_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

# nominal figures of the target (dense, per GPU); measured ones come from MEASURED_PEAKS.json when present
B200_NOMINAL = {"sms": 148, "hbm_gb": 180, "hbm_gbs": 7700.0, "bf16_tflops": 2250.0, "l2_mb": 126,
                "smem_per_cta_kb": 227, "tmem_kb_per_sm": 256, "nvlink_gbs_per_direction": 900.0}


class DeviceType:
    def __init__(self, kind: str, index: int = 0):
        self.kind, self.index = kind, index

    def torch_device(self) -> torch.device:
        return torch.device(self.kind, self.index) if self.kind == "cuda" else torch.device("cpu")

    def is_gpu(self) -> bool:
        return self.kind == "cuda"

    def __repr__(self):
        return "%s:%d" % (self.kind, self.index) if self.is_gpu() else "cpu"


class CPUDevice(DeviceType):
    def __init__(self):
        super().__init__("cpu", 0)


class GPUDevice(DeviceType):
    def __init__(self, index: int = 0):
        super().__init__("cuda", index)


def measured_peaks(path: Optional[str] = None) -> dict:
    """Copy bandwidth and bf16 matmul rate measured on this machine, or the stated fallback."""
    path = path or os.path.join(_ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def describe(device: Optional[DeviceType] = None) -> dict:
    out = {"nominal": dict(B200_NOMINAL), "peaks": measured_peaks()}
    if torch.cuda.is_available():
        idx = device.index if device is not None and device.is_gpu() else torch.cuda.current_device()
        p = torch.cuda.get_device_properties(idx)
        out["device"] = {"name": p.name, "sms": p.multi_processor_count, "memory_gb": p.total_memory / 2 ** 30,
                         "capability": "%d.%d" % (p.major, p.minor)}
    return out
