"""Finite scalar quantisation: each latent channel is squashed to a fixed number of levels and
rounded; the tuple of per-channel levels is one code of an implicit product codebook.

Reference: src/HartsyInference.Core/Codecs/Fsq.cs (codec used by the speech-token models).
"""
from __future__ import annotations

import torch


class Fsq:
    def __init__(self, levels: list[int]):
        self.levels = torch.tensor(levels, dtype=torch.int64)
        self.basis = torch.cumprod(torch.tensor([1] + levels[:-1], dtype=torch.int64), 0)
        self.codebook_size = int(torch.prod(self.levels))

    def bound(self, z: torch.Tensor, eps: float = 1e-3) -> torch.Tensor:
        """Squash channel i into (-(L_i - 1) / 2, (L_i - 1) / 2) (shifted by half a step for even L_i)."""
        lv = self.levels.to(z.device).float()
        half_l = (lv - 1) * (1 + eps) / 2
        offset = torch.where(self.levels.to(z.device) % 2 == 0, 0.5, 0.0)
        shift = torch.atanh(offset / half_l)
        return torch.tanh(z + shift) * half_l - offset

    def quantize(self, z: torch.Tensor) -> torch.Tensor:
        """z [..., d] -> quantised values normalised to [-1, 1]."""
        half_width = (self.levels.to(z.device) // 2).float()
        return torch.round(self.bound(z)) / half_width

    def codes_to_indices(self, zq: torch.Tensor) -> torch.Tensor:
        half_width = (self.levels.to(zq.device) // 2).float()
        digits = torch.round(zq * half_width + half_width).long()
        return (digits * self.basis.to(zq.device)).sum(-1)

    def indices_to_codes(self, idx: torch.Tensor) -> torch.Tensor:
        lv, basis = self.levels.to(idx.device), self.basis.to(idx.device)
        digits = (idx[..., None] // basis) % lv
        half_width = (lv // 2).float()
        return (digits.float() - half_width) / half_width

    def encode(self, z: torch.Tensor) -> torch.Tensor:
        return self.codes_to_indices(self.quantize(z))
