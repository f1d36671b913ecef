"""Flux Redux: a picture as (part of) the prompt. The SigLIP vision states of the picture (729 patch
states of width 1152 for the 384-pixel so400m tower) go through a two-layer projector
(1152 -> 3 x 4096, SiLU, -> 4096) and the resulting tokens are appended to the T5 states of the text,
with text position ids; ``scale`` multiplies them (0 removes the picture's influence short of the
extra attention columns). Weights: ``redux_up.{weight,bias}``, ``redux_down.{weight,bias}``.
Reference: src/HartsyInference.Diffusion/Adapters/ (Redux).
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.nn.functional as F


class ReduxImageEncoder:
    def __init__(self, get: Optional[Callable[[str], Optional[torch.Tensor]]] = None, device="cpu", dtype: torch.dtype = torch.float32,
                 in_dim: int = 1152, txt_dim: int = 4096, seed: int = 0):
        self.device, self.dtype = torch.device(device), dtype
        if get is None:
            g = torch.Generator().manual_seed(seed)
            w = {"redux_up.weight": torch.randn(3 * txt_dim, in_dim, generator=g) * in_dim ** -0.5, "redux_up.bias": torch.zeros(3 * txt_dim),
                 "redux_down.weight": torch.randn(txt_dim, 3 * txt_dim, generator=g) * (3 * txt_dim) ** -0.5, "redux_down.bias": torch.zeros(txt_dim)}
            get = w.get
        self.up = (get("redux_up.weight").to(self.device).to(dtype), get("redux_up.bias").to(self.device).to(dtype))
        self.down = (get("redux_down.weight").to(self.device).to(dtype), get("redux_down.bias").to(self.device).to(dtype))
        self.in_dim, self.txt_dim = self.up[0].shape[1], self.down[0].shape[0]

    @torch.no_grad()
    def __call__(self, states: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
        """vision states [n, in_dim] -> prompt tokens [n, txt_dim]."""
        if states.shape[-1] != self.in_dim:
            raise ValueError(f"vision states of width {states.shape[-1]} for a projector that takes {self.in_dim}")
        x = states.to(self.device).to(self.dtype)
        return F.linear(F.silu(F.linear(x, *self.up)), *self.down) * scale
