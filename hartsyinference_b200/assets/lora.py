"""LoRA adapters, merged into the base weights at load time.

``W' = W + strength * (alpha / rank) * B A`` for every adapted linear; nothing of the adapter
survives into the hot path (weights are re-quantised after the merge when the model runs fp8).
Key styles understood (detected from the tensor names):

* PEFT / diffusers:  ``<module>.lora_A.weight`` / ``<module>.lora_B.weight`` (optionally under
  ``base_model.model.``, with an adapter name segment ``.lora_A.default.weight``)
* kohya:             ``lora_unet_<module_with_underscores>.lora_down.weight`` / ``.lora_up.weight``
  / ``.alpha``; the module path is recovered by matching the flattened name against the base keys
* diffusers (old):   ``<module>.lora.down.weight`` / ``<module>.lora.up.weight``

Reference: src/HartsyInference.ModelAssets/Lora/LoraStack.cs (merge / apply) and its key mappers.
"""
from __future__ import annotations

import re
from dataclasses import dataclass, field
from typing import Callable, Iterable, Optional

import torch


@dataclass
class LoraPair:
    down: torch.Tensor                 # A: [rank, in]
    up: torch.Tensor                   # B: [out, rank]
    alpha: Optional[float] = None

    @property
    def rank(self) -> int:
        return self.down.shape[0]

    def delta(self, strength: float = 1.0) -> torch.Tensor:
        scale = strength * ((self.alpha / self.rank) if self.alpha is not None else 1.0)
        up, down = self.up.float(), self.down.float()
        if down.dim() == 4:            # conv LoRA: 1x1 up over k x k down
            return scale * torch.einsum("or,rikl->oikl", up.flatten(1), down)
        return scale * (up @ down)


_SUFFIXES = [
    (re.compile(r"^(.*)\.lora_A(?:\.[^.]+)?\.weight$"), "down"),
    (re.compile(r"^(.*)\.lora_B(?:\.[^.]+)?\.weight$"), "up"),
    (re.compile(r"^(.*)\.lora_down\.weight$"), "down"),
    (re.compile(r"^(.*)\.lora_up\.weight$"), "up"),
    (re.compile(r"^(.*)\.lora\.down\.weight$"), "down"),
    (re.compile(r"^(.*)\.lora\.up\.weight$"), "up"),
    (re.compile(r"^(.*)\.alpha$"), "alpha"),
]
_PREFIXES = ("base_model.model.", "transformer.", "unet.", "diffusion_model.", "model.diffusion_model.")


def parse_lora(tensors: dict[str, torch.Tensor]) -> dict[str, LoraPair]:
    """Group adapter tensors by the module they adapt (module path as written in the file)."""
    parts: dict[str, dict] = {}
    for name, t in tensors.items():
        for rx, kind in _SUFFIXES:
            m = rx.match(name)
            if m:
                parts.setdefault(m.group(1), {})[kind] = t
                break
    out = {}
    for mod, d in parts.items():
        if "down" in d and "up" in d:
            alpha = float(d["alpha"]) if "alpha" in d else None
            out[mod] = LoraPair(d["down"], d["up"], alpha)
    return out


def _flatten(key: str) -> str:
    return re.sub(r"[^0-9a-zA-Z]", "_", key)


def resolve_targets(modules: Iterable[str], base_keys: Iterable[str]) -> dict[str, str]:
    """Map adapter module paths to base weight keys (``<module>.weight``). Handles optional
    prefixes and kohya's underscore-flattened names."""
    base = [k for k in base_keys if k.endswith(".weight")]
    by_mod = {k[:-len(".weight")]: k for k in base}
    flat = {_flatten(m): k for m, k in by_mod.items()}
    out = {}
    for mod in modules:
        cands = [mod] + [mod[len(p):] for p in _PREFIXES if mod.startswith(p)]
        hit = next((by_mod[c] for c in cands if c in by_mod), None)
        if hit is None:
            f = mod
            for p in ("lora_unet_", "lora_te_", "lora_te1_", "lora_te2_", "lora_transformer_"):
                if f.startswith(p):
                    f = f[len(p):]
                    break
            f = _flatten(f)
            hit = flat.get(f)
            if hit is None:     # the base may carry a prefix the adapter leaves out
                hit = next((k for ff, k in flat.items() if ff.endswith("_" + f)), None)
        if hit is not None:
            out[mod] = hit
    return out


@dataclass
class LoraStack:
    """Several adapters with strengths, applied as one merged delta per weight."""
    adapters: list[tuple[dict[str, LoraPair], float]] = field(default_factory=list)

    def add(self, tensors: dict[str, torch.Tensor], strength: float = 1.0) -> "LoraStack":
        self.adapters.append((parse_lora(tensors), strength))
        return self

    def wrap(self, get: Callable[[str], Optional[torch.Tensor]], base_keys: Iterable[str]) -> Callable[[str], Optional[torch.Tensor]]:
        """Returns a ``get(name)`` that yields merged weights; loaders keep slicing / quantising as
        before and never see the adapter."""
        keys = list(base_keys)
        plans: dict[str, list[tuple[LoraPair, float]]] = {}
        self.unmatched: list[str] = []
        for pairs, strength in self.adapters:
            targets = resolve_targets(pairs.keys(), keys)
            for mod, pair in pairs.items():
                if mod in targets:
                    plans.setdefault(targets[mod], []).append((pair, strength))
                else:
                    self.unmatched.append(mod)

        def merged(name: str) -> Optional[torch.Tensor]:
            w = get(name)
            if w is None or name not in plans:
                return w
            acc = w.float()
            for pair, strength in plans[name]:
                d = pair.delta(strength)
                if d.shape != acc.shape:
                    raise ValueError(f"LoRA delta {tuple(d.shape)} does not fit {name} {tuple(acc.shape)}")
                acc = acc + d
            return acc.to(w.dtype)

        return merged
