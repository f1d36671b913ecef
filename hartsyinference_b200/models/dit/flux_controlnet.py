"""Flux ControlNet: a shallow copy of the Flux transformer (a few double and single blocks) that
also embeds a control image's latents, runs its blocks on [text | image + control] and projects the
image stream after each block through a zero-initialised linear layer. The projections are added to
the base model's image stream after the blocks they map to, scaled by the conditioning strength.

Reference: src/HartsyInference.Diffusion/Adapters/ (FluxControlNet). Tensor names follow diffusers
``FluxControlNetModel`` (``controlnet_x_embedder``, ``controlnet_blocks.N``,
``controlnet_single_blocks.N`` beside the transformer's own names).
"""
from __future__ import annotations

from typing import Callable, Optional

import torch

from ... import ops
from .common import WeightFactory
from .flux import FluxConfig, FluxTransformer


class FluxControlNet(FluxTransformer):
    def __init__(self, cfg: FluxConfig, device="cpu", fp8: bool = False,
                 get: Optional[Callable[[str], Optional[torch.Tensor]]] = None, seed: int = 0):
        # the branch has no output head (no norm_out / proj_out in its checkpoint)
        super().__init__(cfg, device, fp8=fp8, get=get, seed=seed, build_head=False)
        f = WeightFactory(self.device, False, get=get, seed=seed + 101)
        H = cfg.hidden_size
        self.control_embedder = f.linear("controlnet_x_embedder", H, cfg.in_channels, allow_fp8=False)
        self.double_proj = [f.linear(f"controlnet_blocks.{i}", H, H, allow_fp8=False) for i in range(cfg.num_double_blocks)]
        self.single_proj = [f.linear(f"controlnet_single_blocks.{i}", H, H, allow_fp8=False) for i in range(cfg.num_single_blocks)]

    @torch.no_grad()
    def residuals(self, img: torch.Tensor, control: torch.Tensor, txt: torch.Tensor, timestep: torch.Tensor, pooled: torch.Tensor,
                  img_ids: torch.Tensor, txt_ids: torch.Tensor, guidance: Optional[torch.Tensor] = None, scale: float = 1.0):
        """img / control [1, S_i, C_in] packed latents -> (double residuals, single residuals) for
        ``FluxTransformer.forward(control=...)``."""
        dt = torch.bfloat16
        B, S_i = img.shape[0], img.shape[1]
        if B != 1:
            raise ValueError("the ControlNet branch runs one sample at a time")
        x_i = ops.linear(img.reshape(S_i, -1).to(dt), self.x_embedder)
        x_i = (x_i.float() + ops.linear(control.reshape(S_i, -1).to(self.device).to(dt), self.control_embedder).float()).to(dt)
        x_t = ops.linear(txt.reshape(txt.shape[1], -1).to(dt), self.context_embedder)
        doubles, singles = [], []
        super().forward(img, txt, timestep, pooled, img_ids, txt_ids, guidance, hidden_in=(x_i, x_t, None), collect=(doubles, singles))
        out_d = [(ops.linear(h.contiguous(), w).float() * scale).to(dt) for h, w in zip(doubles, self.double_proj)]
        out_s = [(ops.linear(h.contiguous(), w).float() * scale).to(dt) for h, w in zip(singles, self.single_proj)]
        return out_d, out_s
