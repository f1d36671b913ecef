"""PyTorch ``.pt`` / ``.pth`` / ``.bin`` / ``.ckpt`` checkpoints as a flat ``{name: tensor}`` map.

Loading goes through ``torch.load(weights_only=True)``: the restricted unpickler that builds tensors
and plain containers only, so a checkpoint cannot run code. Zip-format files are memory-mapped.
Common wrappers (``state_dict``, ``model``, ``module``, ``ema``, nested dicts) are flattened.

Reference: src/HartsyInference.ModelAssets/ (PyTorch pickle-zip tensor reader).
"""
from __future__ import annotations

import zipfile
from pathlib import Path

import torch

_WRAPPERS = ("state_dict", "model", "module", "model_state_dict", "net", "params", "params_ema", "generator", "weight")


def _flatten(obj, prefix: str, out: dict[str, torch.Tensor]) -> None:
    if isinstance(obj, torch.Tensor):
        out[prefix.rstrip(".")] = obj
    elif isinstance(obj, dict):
        for k, v in obj.items():
            _flatten(v, f"{prefix}{k}.", out)
    elif isinstance(obj, (list, tuple)):
        for i, v in enumerate(obj):
            _flatten(v, f"{prefix}{i}.", out)


def load_torch_checkpoint(path, unwrap: bool = True) -> dict[str, torch.Tensor]:
    p = Path(path)
    mmap = zipfile.is_zipfile(p)
    obj = torch.load(p, map_location="cpu", weights_only=True, mmap=mmap)
    while unwrap and isinstance(obj, dict):
        inner = next((obj[k] for k in _WRAPPERS if isinstance(obj.get(k), dict)
                      and not any(isinstance(v, torch.Tensor) for v in obj.values())), None)
        if inner is None:
            break
        obj = inner
    out: dict[str, torch.Tensor] = {}
    _flatten(obj, "", out)
    return out
