"""Checkpoints in the variable layout of the reference's TensorFlow ResNet.

Names follow the reference's scope and TF-layers auto-numbering in creation order
(official/resnet/resnet_model.py:486,97-101,55-60,552; golden checkpoints under
official/utils/testing/reference_data/resnet/*/model.ckpt.index):

    resnet_model/conv2d[_k]/kernel                                   HWIO
    resnet_model/batch_normalization[_k]/{gamma,beta,moving_mean,moving_variance}
    resnet_model/dense/{kernel,bias}                                 kernel is [in, out]
    <variable>/Momentum                                              one slot per trainable variable
    global_step

fp32 master values are exported even when the model computes in bf16.  TensorFlow is not
available here, so the container is a ``.npz`` archive (name -> array); the names and array
layouts are what a TF-side converter needs.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch
import torch.nn as nn


def _suffix(k: int) -> str:
    return "" if k == 0 else "_%d" % k


def tf_variables(model: nn.Module, scope: str = "resnet_model") -> List[Tuple[str, torch.Tensor, str]]:
    """(tf name, tensor, kind) in creation order; kind in {conv, gamma, beta, mean, var, dense_w, dense_b}."""
    pre = scope + "/" if scope else ""
    out, nconv, nbn, ndense = [], 0, 0, 0
    for kind, mod in model.registry:
        if kind == "conv":
            out.append(("%sconv2d%s/kernel" % (pre, _suffix(nconv)), mod.weight, "conv"))
            nconv += 1
        elif kind == "bn":
            base = "%sbatch_normalization%s/" % (pre, _suffix(nbn))
            out += [(base + "gamma", mod.weight, "gamma"), (base + "beta", mod.bias, "beta"),
                    (base + "moving_mean", mod.running_mean, "mean"), (base + "moving_variance", mod.running_var, "var")]
            nbn += 1
        elif kind == "dense":
            base = "%sdense%s/" % (pre, _suffix(ndense))
            out += [(base + "kernel", mod.weight, "dense_w"), (base + "bias", mod.bias, "dense_b")]
            ndense += 1
    return out


def _to_tf(t: torch.Tensor, kind: str) -> np.ndarray:
    a = t.detach().float().cpu()
    if kind == "conv":
        a = a.permute(2, 3, 1, 0)      # OIHW -> HWIO
    elif kind == "dense_w":
        a = a.t()                      # [out, in] -> [in, out]
    return a.contiguous().numpy()


def _from_tf(a: np.ndarray, kind: str) -> torch.Tensor:
    t = torch.from_numpy(np.ascontiguousarray(a))
    if kind == "conv":
        t = t.permute(3, 2, 0, 1)
    elif kind == "dense_w":
        t = t.t()
    return t.contiguous()


def export_tf_layout(model: nn.Module, path: str, optimizer=None, global_step: int = 0,
                     scope: str = "resnet_model") -> Dict[str, np.ndarray]:
    """Write ``path`` (.npz) with every variable, its Momentum slot (when ``optimizer`` is given:
    an eager-SGD wrapper or a torch SGD) and ``global_step``.  Returns the dict written."""
    master = {}
    momentum = {}
    if optimizer is not None and hasattr(optimizer, "master_params"):
        master = {id(p): m for p, m in optimizer.master_params()}
        momentum = {id(p): b for p, b in optimizer.momentum_buffers() if b is not None}
    elif optimizer is not None:
        for g in optimizer.param_groups:
            for p in g["params"]:
                buf = optimizer.state.get(p, {}).get("momentum_buffer")
                if buf is not None:
                    momentum[id(p)] = buf
    arrays: Dict[str, np.ndarray] = {}
    for name, t, kind in tf_variables(model, scope):
        src = master.get(id(t), t)
        arrays[name] = _to_tf(src, kind)
        if kind not in ("mean", "var") and optimizer is not None:
            buf = momentum.get(id(t))
            arrays[name + "/Momentum"] = _to_tf(buf, kind) if buf is not None else np.zeros_like(arrays[name])
    arrays["global_step"] = np.asarray(global_step, dtype=np.int64)
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    np.savez(path, **arrays)
    return arrays


def import_tf_layout(model: nn.Module, path: str, scope: str = "resnet_model", exclude: Tuple[str, ...] = ()) -> int:
    """Load variables by name; ``exclude`` skips name substrings (warm start without ``dense``,
    as the reference's ``--pretrained_model_checkpoint_path`` does).  Returns global_step."""
    z = np.load(path if path.endswith(".npz") else path + ".npz")
    with torch.no_grad():
        for name, t, kind in tf_variables(model, scope):
            if any(x in name for x in exclude) or name not in z:
                continue
            t.copy_(_from_tf(z[name], kind).to(t.device, t.dtype))
    return int(z["global_step"]) if "global_step" in z else 0


# ------------------------------------------------------------------ per-rank training state
def save(model: nn.Module, optimizer, model_dir: str, rank: int, global_step: int, extra: Optional[dict] = None):
    """Every rank writes its own directory ``<model_dir>/<rank>`` (the reference gives each rank
    its own Estimator model_dir, resnet_run_loop_solo_imagenet_300.py:551-556)."""
    d = os.path.join(model_dir, str(rank))
    os.makedirs(d, exist_ok=True)
    state = {"model": model.state_dict(), "global_step": global_step, "extra": extra or {}}
    if optimizer is not None:
        state["optimizer"] = optimizer.state_dict()
    tmp = os.path.join(d, "ckpt-%d.pt.tmp" % global_step)
    torch.save(state, tmp)
    os.replace(tmp, os.path.join(d, "ckpt-%d.pt" % global_step))
    with open(os.path.join(d, "checkpoint"), "w") as f:
        json.dump({"latest": "ckpt-%d.pt" % global_step, "global_step": global_step}, f)
    return d


def latest(model_dir: str, rank: int) -> Optional[str]:
    d = os.path.join(model_dir, str(rank))
    idx = os.path.join(d, "checkpoint")
    if not os.path.exists(idx):
        return None
    return os.path.join(d, json.load(open(idx))["latest"])


def load(model: nn.Module, optimizer, model_dir: str, rank: int) -> int:
    """Resume from the latest checkpoint of this rank's directory; returns global_step (0 if none)."""
    path = latest(model_dir, rank)
    if path is None:
        return 0
    state = torch.load(path, map_location="cpu", weights_only=False)
    with torch.no_grad():
        own = model.state_dict()
        for k, v in state["model"].items():
            if k in own:
                own[k].copy_(v.to(own[k].device, own[k].dtype))
    if optimizer is not None and "optimizer" in state:
        optimizer.load_state_dict(state["optimizer"])
    elif optimizer is not None and hasattr(optimizer, "refresh_master_from_params"):
        optimizer.refresh_master_from_params()   # a model-only checkpoint: master weights follow the parameters
    return int(state["global_step"])


def clean(model_dir: str):
    """``--clean``: remove a model directory (official/utils/misc/model_helpers.py:89-93)."""
    import shutil
    if os.path.isdir(model_dir):
        shutil.rmtree(model_dir)


def resync_from_rank0(model: nn.Module, optimizer, group) -> None:
    """Make every replica equal to rank 0's: weights, momentum and batch-norm statistics.
    In-job replacement for copying rank 0's checkpoint directory over the others between
    launches (official/resnet/test_scripts_imagenet/synchm.sh:4-12)."""
    if group.world == 1:
        return
    if optimizer is not None and hasattr(optimizer, "resync_from_rank0"):
        optimizer.resync_from_rank0()
    else:
        for p in model.parameters():
            group.bcast(p.data)
    for b in model.buffers():
        if b.is_floating_point():
            group.bcast(b)
