"""CLIPSeg: text-prompted segmentation on top of CLIP.

The CLIP vision tower's token states are tapped after a few blocks; starting from the deepest tap,
each is reduced to a small width and added to the running state, the first one is modulated by the
prompt's CLIP text embedding (FiLM: scale and shift), and a small post-LayerNorm transformer layer
follows each tap. The class token is dropped, the patch grid is upsampled to the input size by one
transposed convolution, and the result is a logit map (sigmoid = mask probability).

Reference: src/HartsyInference.Vision/ (ClipSeg segmenter behind the vision service's segment
operation). Tensor names follow Hugging Face ``CLIPSegForImageSegmentation`` (``clip.*``, ``decoder.*``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.nn.functional as F

from ..encoders.clip import ClipTextConfig, ClipTextEncoder, clip_text_from_hf
from ..encoders.clip_vision import ClipVisionConfig, ClipVisionEncoder, clip_vision_from_hf


@dataclass(frozen=True)
class ClipSegConfig:
    vision: ClipVisionConfig
    text: ClipTextConfig
    projection_dim: int = 512
    extract_layers: tuple = (3, 6, 9)
    reduce_dim: int = 64
    decoder_heads: int = 4
    decoder_ffn: int = 2048
    conditional_layer: int = 0


def clipseg_from_hf(d: dict) -> ClipSegConfig:
    return ClipSegConfig(vision=clip_vision_from_hf(d["vision_config"]), text=clip_text_from_hf(d["text_config"]),
                         projection_dim=d.get("projection_dim", 512), extract_layers=tuple(d.get("extract_layers", (3, 6, 9))),
                         reduce_dim=d.get("reduce_dim", 64), decoder_heads=d.get("decoder_num_attention_heads", 4),
                         decoder_ffn=d.get("decoder_intermediate_size", 2048), conditional_layer=d.get("conditional_layer", 0))


class ClipSeg:
    def __init__(self, cfg: ClipSegConfig, device="cpu", get: Optional[Callable[[str], Optional[torch.Tensor]]] = None, seed: int = 0):
        self.cfg, self.device = cfg, torch.device(device)
        sub = None if get is None else (lambda n: get("clip." + n))
        self.vision = ClipVisionEncoder(cfg.vision, device, get=sub, seed=seed, prefix="vision_model.")
        self.text = ClipTextEncoder(cfg.text, device, get=sub, seed=seed + 1)
        self._get = get
        self._g = torch.Generator().manual_seed(seed + 2)
        self.w: dict[str, torch.Tensor] = {}
        if get is None:      # synthetic: a text projection of the right shape
            self.text.projection = torch.randn(cfg.projection_dim, cfg.text.width, generator=self._g).to(self.device) * 0.05

    def _p(self, name: str, *shape) -> torch.Tensor:
        t = self.w.get(name)
        if t is None:
            t = self._get("decoder." + name) if self._get is not None else None
            if t is None:
                if self._get is not None:
                    raise KeyError("decoder." + name)
                fan = shape[-1] if len(shape) > 1 else 1
                t = torch.zeros(*shape) if name.endswith("bias") else torch.randn(*shape, generator=self._g) * (1.0 / fan) ** 0.5
            t = t.float().to(self.device)
            self.w[name] = t
        return t

    def _lin(self, x, name, o, i):
        return F.linear(x, self._p(name + ".weight", o, i), self._p(name + ".bias", o))

    @torch.no_grad()
    def text_embedding(self, ids: torch.Tensor) -> torch.Tensor:
        """The prompt's projected CLIP text feature [projection_dim] (not normalised)."""
        return self.text.encode(ids, project=True)[1].float()

    @torch.no_grad()
    def segment(self, image: torch.Tensor, cond: torch.Tensor) -> torch.Tensor:
        """image [3, S, S] normalised with CLIP statistics, cond [projection_dim] -> logits [S, S]."""
        cfg = self.cfg
        R, h = cfg.reduce_dim, cfg.decoder_heads
        W = cfg.vision.width
        taps = [self.vision.hidden_states(image, layer=i + 1).float() for i in cfg.extract_layers][::-1]
        cond = cond.to(self.device).float()
        out = None
        for i, act in enumerate(taps):
            red = self._lin(act, f"reduces.{i}", R, W)
            out = red if out is None else red + out
            if i == cfg.conditional_layer:
                out = self._lin(cond, "film_mul", R, cfg.projection_dim) * out + self._lin(cond, "film_add", R, cfg.projection_dim)
            p = f"layers.{i}."
            T = out.shape[0]
            q, k, v = (self._lin(out, p + f"self_attn.{n}_proj", R, R).reshape(T, h, R // h).transpose(0, 1) for n in ("q", "k", "v"))
            a = F.scaled_dot_product_attention(q[None], k[None], v[None])[0].transpose(0, 1).reshape(T, R)
            out = F.layer_norm(out + self._lin(a, p + "self_attn.out_proj", R, R), (R,), self._p(p + "layer_norm1.weight", R),
                               self._p(p + "layer_norm1.bias", R), 1e-5)
            m = self._lin(torch.relu(self._lin(out, p + "mlp.fc1", cfg.decoder_ffn, R)), p + "mlp.fc2", R, cfg.decoder_ffn)
            out = F.layer_norm(out + m, (R,), self._p(p + "layer_norm2.weight", R), self._p(p + "layer_norm2.bias", R), 1e-5)
        side = int(round((out.shape[0] - 1) ** 0.5))
        fmap = out[1:].t().reshape(1, R, side, side)
        P = cfg.vision.patch
        up = F.conv_transpose2d(fmap, self._p("transposed_convolution.weight", R, 1, P, P), self._p("transposed_convolution.bias", 1), stride=P)
        return up[0, 0]
