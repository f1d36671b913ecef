"""Chroma: a Flux-architecture transformer whose per-block AdaLN vectors come from one small
"approximator" network instead of a modulation linear in every block.

For a timestep, the approximator embeds (timestep, a constant zero guidance) and the index of every
modulation slot (3 per single block, 6 per image and per text stream of each double block, 2 for the
output norm), runs a residual MLP with RMSNorm over all slots at once, and each block looks its
vectors up by slot. There is no pooled-text or guidance conditioning; the blocks themselves (joint
attention with rotary embedding, fused single blocks) are Flux's and run on the same kernels.

Reference: src/HartsyInference.Diffusion/Models/Denoisers/ChromaTransformer.cs, ChromaConfig.cs.
Tensor names follow diffusers ``ChromaTransformer2DModel`` (``distilled_guidance_layer.*`` beside
the Flux block names).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.nn.functional as F

from .common import WeightFactory, timestep_embedding
from .flux import FluxConfig, FluxTransformer


@dataclass(frozen=True)
class ChromaConfig(FluxConfig):
    num_double_blocks: int = 19
    num_single_blocks: int = 38
    guidance_embed: bool = False
    approximator_channels: int = 64
    approximator_hidden: int = 5120
    approximator_layers: int = 5

    @property
    def mod_slots(self) -> int:
        return 3 * self.num_single_blocks + 12 * self.num_double_blocks + 2


def tiny_chroma(**over) -> ChromaConfig:
    kw = dict(in_channels=16, hidden_size=128, num_heads=4, head_dim=32, num_double_blocks=2, num_single_blocks=2,
              context_dim=64, pooled_dim=32, axes_dim=(8, 12, 12), approximator_channels=16, approximator_hidden=48, approximator_layers=2)
    kw.update(over)
    return ChromaConfig(**kw)


class ChromaTransformer(FluxTransformer):
    HAS_MODULATION_LINEARS = False

    def __init__(self, cfg: ChromaConfig, device="cpu", comm=None, fp8: bool = False,
                 get: Optional[Callable[[str], Optional[torch.Tensor]]] = None, seed: int = 0):
        super().__init__(cfg, device, comm=comm, fp8=fp8, get=get, seed=seed)
        f = WeightFactory(self.device, False, get=get, seed=seed + 31)
        a, hd, H = cfg.approximator_channels, cfg.approximator_hidden, cfg.hidden_size
        p = "distilled_guidance_layer."
        t32 = lambda name, *shape, **kw: f.tensor(name, *shape, **kw).float()
        self.ap_in = (t32(p + "in_proj.weight", hd, a), t32(p + "in_proj.bias", hd, zeros=True))
        self.ap_layers = [dict(norm=t32(f"{p}norms.{i}.weight", hd, ones=True),
                               w1=t32(f"{p}layers.{i}.linear_1.weight", hd, hd), b1=t32(f"{p}layers.{i}.linear_1.bias", hd, zeros=True),
                               w2=t32(f"{p}layers.{i}.linear_2.weight", hd, hd), b2=t32(f"{p}layers.{i}.linear_2.bias", hd, zeros=True))
                          for i in range(cfg.approximator_layers)]
        self.ap_out = (t32(p + "out_proj.weight", H, hd), t32(p + "out_proj.bias", H, zeros=True))
        # the slot-index embedding is a constant of the architecture
        idx = torch.arange(cfg.mod_slots, dtype=torch.float32) * 1000.0
        self.slot_embed = timestep_embedding(idx, a // 2).to(self.device)             # [slots, a / 2]
        self._mods: Optional[torch.Tensor] = None

    def modulations(self, timestep: torch.Tensor) -> torch.Tensor:
        """sigma [B] -> every modulation vector [B, slots, H] (fp32)."""
        cfg = self.cfg
        a = cfg.approximator_channels
        t = timestep_embedding(timestep.to(self.device) * 1000.0, a // 4)
        g = timestep_embedding(torch.zeros_like(timestep, device=self.device), a // 4)
        tg = torch.cat([t, g], 1)[:, None, :].expand(-1, cfg.mod_slots, -1)
        x = torch.cat([tg, self.slot_embed[None].expand(tg.shape[0], -1, -1)], -1)     # [B, slots, a]
        x = F.linear(x, *self.ap_in)
        for lw in self.ap_layers:
            y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * lw["norm"]
            x = x + F.linear(F.silu(F.linear(y, lw["w1"], lw["b1"])), lw["w2"], lw["b2"])
        return F.linear(x, *self.ap_out)

    def time_embedding(self, timestep, guidance, pooled):
        # called once at the top of forward: the place to compute this step's modulation table
        self._mods = self.modulations(timestep)
        return torch.zeros(timestep.shape[0], self.cfg.hidden_size, dtype=torch.bfloat16, device=self.device)

    def _slot(self, kind: str, index: int) -> tuple[int, int]:
        cfg = self.cfg
        if kind == "single":
            return 3 * index, 3
        base = 3 * cfg.num_single_blocks + (6 * cfg.num_double_blocks if kind == "txt" else 0)
        return base + 6 * index, 6

    def _mod(self, temb_act, w, kind: str, index: int) -> torch.Tensor:
        s, n = self._slot(kind, index)
        return self._mods[:, s:s + n].reshape(self._mods.shape[0], -1).to(torch.bfloat16)

    def _final_mod(self, temb_act) -> torch.Tensor:
        # the last two slots are (shift, scale); the shared output path wants (scale, shift)
        m = self._mods[:, -2:]
        return torch.cat([m[:, 1], m[:, 0]], -1).to(torch.bfloat16)
