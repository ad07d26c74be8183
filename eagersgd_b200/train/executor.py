"""Network and executor abstractions over PyTorch modules.

``Network`` exposes parameters, gradients and tensors by name (deep500/lv1/network.py:19-89)
and ``GraphExecutor`` runs ``inference`` / ``inference_and_backprop`` with executor events
(deep500/lv1/graph_executor.py:8-32; PyTorch flavour deep500/frameworks/pytorch/
pytorch_graph_executor.py:87-173).  PyTorch is the only framework layer here, so there is
one implementation instead of one per backend.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.nn as nn


class Network:
    def __init__(self, module: nn.Module, device: Optional[torch.device] = None):
        self.module = module
        self.device = device or next(module.parameters()).device
        self._feeds: Dict[str, torch.Tensor] = {}

    # ---- parameters ---------------------------------------------------------
    def get_params(self) -> List[str]:
        return [n for n, p in self.module.named_parameters() if p.requires_grad]

    def _param(self, name: str) -> nn.Parameter:
        return dict(self.module.named_parameters())[name]

    def fetch_tensor(self, name: str) -> np.ndarray:
        if name in self._feeds:
            return self._feeds[name].detach().float().cpu().numpy()
        sd = dict(self.module.named_parameters())
        sd.update(dict(self.module.named_buffers()))
        return sd[name].detach().float().cpu().numpy()

    def fetch_tensors(self, names: Sequence[str]) -> List[np.ndarray]:
        return [self.fetch_tensor(n) for n in names]

    def feed_tensor(self, name: str, value, device_option=None) -> None:
        sd = dict(self.module.named_parameters())
        sd.update(dict(self.module.named_buffers()))
        t = torch.as_tensor(value)
        if name in sd:
            with torch.no_grad():
                sd[name].copy_(t.to(sd[name].device, sd[name].dtype))
        else:
            self._feeds[name] = t.to(self.device)

    def gradient(self) -> List[Tuple[str, str]]:
        """(parameter name, gradient name) pairs."""
        return [(n, n + ".grad") for n in self.get_params()]

    def fetch_gradient(self, name: str) -> Optional[np.ndarray]:
        g = self._param(name).grad
        return None if g is None else g.detach().float().cpu().numpy()

    def get_input_nodes(self) -> List[str]:
        return ["x"]

    def get_output_nodes(self) -> List[str]:
        return ["output"]

    def add_output(self, name: str):
        pass

    def export_native(self, path: str, inputs=None):
        torch.save(self.module.state_dict(), path)


class GraphExecutor:
    """Runs a module; ``loss_fn(outputs, batch) -> scalar`` defines the training objective."""

    def __init__(self, module: nn.Module, loss_fn: Optional[Callable] = None, device: Optional[torch.device] = None,
                 events: Optional[Sequence] = None, data_node: str = "x", label_node: str = "y",
                 input_dtype: Optional[torch.dtype] = None, channels_last: bool = False):
        self.network = Network(module, device)
        self.module = module
        self.device = self.network.device
        self.loss_fn = loss_fn
        self.events = list(events or [])
        self.data_node, self.label_node = data_node, label_node
        self.input_dtype, self.channels_last = input_dtype, channels_last

    def _to_device(self, batch: Dict) -> Dict[str, torch.Tensor]:
        out = {}
        for k, v in batch.items():
            t = v if isinstance(v, torch.Tensor) else torch.as_tensor(np.asarray(v))
            t = t.to(self.device, non_blocking=True)
            if k == self.data_node:
                if self.input_dtype is not None and t.is_floating_point():
                    t = t.to(self.input_dtype)
                if self.channels_last and t.dim() == 4:
                    t = t.contiguous(memory_format=torch.channels_last)
            out[k] = t
        return out

    def _fire(self, hook: str, *args):
        for e in self.events:
            fn = getattr(e, hook, None)
            if fn is not None:
                fn(*args)

    def inference(self, batch: Dict) -> Dict[str, torch.Tensor]:
        self._fire("before_executor", batch)
        b = self._to_device(batch)
        was_training = self.module.training
        self.module.eval()
        with torch.no_grad():
            out = self.module(b[self.data_node])
        self.module.train(was_training)
        res = {"output": out}
        if self.loss_fn is not None and self.label_node in b:
            res["loss"] = self.loss_fn(out, b)
        self._fire("after_inference", res)
        return res

    def inference_and_backprop(self, batch: Dict, loss_name: str = "loss") -> Dict[str, torch.Tensor]:
        self._fire("before_executor", batch)
        b = self._to_device(batch)
        self.module.train()
        out = self.module(b[self.data_node])
        res = {"output": out}
        self._fire("after_inference", res)
        loss = self.loss_fn(out, b)
        loss.backward()
        res[loss_name] = loss.detach()
        self._fire("after_backprop", res)
        return res


def classification_loss(outputs: torch.Tensor, batch: Dict[str, torch.Tensor]) -> torch.Tensor:
    from ..ops.functional import softmax_cross_entropy
    return softmax_cross_entropy(outputs if outputs.dtype == torch.float32 else outputs.float(), batch["y"])


def mse_loss(outputs: torch.Tensor, batch: Dict[str, torch.Tensor]) -> torch.Tensor:
    return torch.nn.functional.mse_loss(outputs.float(), batch["y"].float())


def from_model(module: nn.Module, device=None, loss_fn: Optional[Callable] = classification_loss, events=None,
               data_node: str = "x", label_node: str = "y", **kw) -> GraphExecutor:
    """An executor around a ``torch.nn.Module`` on ``device`` (a ``torch.device``, a device descriptor of
    ``utils.device`` or None for the GPU if there is one) — what recipes name as their ``executor``
    (the reference's ``d5fw.from_model``, deep500/frameworks/pytorch/__init__.py)."""
    if device is not None and not isinstance(device, torch.device):
        device = device.torch_device() if hasattr(device, "torch_device") else torch.device(str(device))
    if device is not None and device.type == "cuda" and not torch.cuda.is_available():
        import warnings
        warnings.warn("no CUDA device here: the executor runs on the CPU")
        device = torch.device("cpu")
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    return GraphExecutor(module.to(device), loss_fn, device=device, events=events, data_node=data_node,
                         label_node=label_node, **kw)
