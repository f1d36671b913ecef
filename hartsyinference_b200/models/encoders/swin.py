"""Swin Transformer backbone: hierarchical feature maps at strides 4, 8, 16, 32 for detection and
segmentation heads (Grounding DINO, UperNet).

A 4 x 4 patch convolution + LayerNorm, then four stages of blocks; a block is LayerNorm, attention
inside non-overlapping ``window x window`` tiles (every second block on a grid rolled by half a
window, with a mask that keeps tokens from different sides of the roll apart), a learned bias per
relative offset and head, and a GELU MLP. Maps whose sides are not multiples of the window are
zero-padded for the attention and cropped after it. Between stages 2 x 2 neighbourhoods are
concatenated (4 C), normalised and reduced to 2 C. Every requested stage output gets its own
LayerNorm. Weights by the `transformers` ``SwinBackbone`` names.
Reference: src/HartsyInference.Vision/Detection/GroundingDino/ (Swin backbone).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.nn.functional as F


@dataclass(frozen=True)
class SwinConfig:
    embed_dim: int = 96
    depths: tuple = (2, 2, 6, 2)
    heads: tuple = (3, 6, 12, 24)
    window: int = 7
    patch: int = 4
    mlp_ratio: float = 4.0
    channels: int = 3
    eps: float = 1e-5
    out_stages: tuple = (2, 3, 4)            # 1-based stage numbers whose maps are returned

    @staticmethod
    def from_hf(d: dict) -> "SwinConfig":
        depths = tuple(d.get("depths", (2, 2, 6, 2)))
        feats = d.get("out_features") or [f"stage{i}" for i in d.get("out_indices", range(1, len(depths) + 1)) if i > 0]
        return SwinConfig(embed_dim=d.get("embed_dim", 96), depths=depths, heads=tuple(d.get("num_heads", (3, 6, 12, 24))),
                          window=d.get("window_size", 7), patch=d.get("patch_size", 4), mlp_ratio=d.get("mlp_ratio", 4.0),
                          channels=d.get("num_channels", 3), eps=d.get("layer_norm_eps", 1e-5),
                          out_stages=tuple(int(f.replace("stage", "")) for f in feats if f != "stem"))


class SwinBackbone:
    def __init__(self, cfg: SwinConfig, get: Callable[[str], Optional[torch.Tensor]], device="cpu", dtype: torch.dtype = torch.float32,
                 prefix: str = ""):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        self._get, self._prefix, self._cache = get, prefix, {}
        w = cfg.window
        coords = torch.stack(torch.meshgrid(torch.arange(w), torch.arange(w), indexing="ij")).flatten(1)
        rel = (coords[:, :, None] - coords[:, None, :]).permute(1, 2, 0) + (w - 1)
        self._rel_index = (rel[..., 0] * (2 * w - 1) + rel[..., 1]).to(self.device)          # [w*w, w*w]

    def _w(self, name: str, optional: bool = False):
        hit = self._cache.get(name, False)
        if hit is False:
            t = self._get(self._prefix + name)
            if t is None and not optional:
                raise KeyError(self._prefix + name)
            hit = None if t is None else t.to(self.device).to(self.dtype)
            self._cache[name] = hit
        return hit

    def _ln(self, x, p: str):
        return F.layer_norm(x, (x.shape[-1],), self._w(p + ".weight"), self._w(p + ".bias"), self.cfg.eps)

    def _lin(self, x, p: str):
        return F.linear(x, self._w(p + ".weight"), self._w(p + ".bias", True))

    def _shift_mask(self, h: int, w: int, shift: int) -> torch.Tensor:
        ws = self.cfg.window
        img = torch.zeros(h, w, device=self.device)
        n = 0
        for hs in (slice(0, -ws), slice(-ws, -shift), slice(-shift, None)):
            for wsl in (slice(0, -ws), slice(-ws, -shift), slice(-shift, None)):
                img[hs, wsl] = n
                n += 1
        win = img.view(h // ws, ws, w // ws, ws).permute(0, 2, 1, 3).reshape(-1, ws * ws)
        return (win[:, None, :] != win[:, :, None]).to(self.dtype) * -100.0                  # [windows, ws*ws, ws*ws]

    def _block(self, x, h: int, w: int, p: str, heads: int, shift: int):
        ws = self.cfg.window
        b, _, c = x.shape
        y = self._ln(x, p + ".layernorm_before").view(b, h, w, c)
        pr, pb = (ws - w % ws) % ws, (ws - h % ws) % ws
        if pr or pb:
            y = F.pad(y, (0, 0, 0, pr, 0, pb))
        hp, wp = h + pb, w + pr
        if shift:
            y = torch.roll(y, (-shift, -shift), (1, 2))
        win = y.view(b, hp // ws, ws, wp // ws, ws, c).permute(0, 1, 3, 2, 4, 5).reshape(-1, ws * ws, c)
        d = c // heads
        split = lambda t: t.view(t.shape[0], ws * ws, heads, d).transpose(1, 2)
        q, k, v = (split(self._lin(win, f"{p}.attention.self.{n}")) for n in ("query", "key", "value"))
        bias = self._w(p + ".attention.self.relative_position_bias_table")[self._rel_index.view(-1)].view(ws * ws, ws * ws, heads).permute(2, 0, 1)
        mask = bias[None]
        if shift:
            m = self._shift_mask(hp, wp, shift)                                               # one per window position
            mask = mask + m[:, None].repeat(b, 1, 1, 1)
        a = F.scaled_dot_product_attention(q, k, v, attn_mask=mask.to(q.dtype)).transpose(1, 2).reshape(-1, ws * ws, c)
        a = self._lin(a, p + ".attention.output.dense")
        a = a.view(b, hp // ws, wp // ws, ws, ws, c).permute(0, 1, 3, 2, 4, 5).reshape(b, hp, wp, c)
        if shift:
            a = torch.roll(a, (shift, shift), (1, 2))
        if pr or pb:
            a = a[:, :h, :w].contiguous()
        x = x + a.view(b, h * w, c)
        y = self._lin(F.gelu(self._lin(self._ln(x, p + ".layernorm_after"), p + ".intermediate.dense")), p + ".output.dense")
        return x + y

    def _merge(self, x, h: int, w: int, p: str):
        b, _, c = x.shape
        y = x.view(b, h, w, c)
        if h % 2 or w % 2:
            y = F.pad(y, (0, 0, 0, w % 2, 0, h % 2))
        y = torch.cat([y[:, 0::2, 0::2], y[:, 1::2, 0::2], y[:, 0::2, 1::2], y[:, 1::2, 1::2]], -1)
        y = y.view(b, -1, 4 * c)
        return F.linear(self._ln(y, p + ".norm"), self._w(p + ".reduction.weight"))

    @torch.no_grad()
    def __call__(self, pixels: torch.Tensor) -> list:
        """pixels [B, 3, H, W] (normalised) -> feature maps [B, C_s, H / stride_s, W / stride_s] of ``cfg.out_stages``."""
        cfg = self.cfg
        x = pixels.to(self.device).to(self.dtype)
        ph, pw = (-x.shape[-2]) % cfg.patch, (-x.shape[-1]) % cfg.patch
        if ph or pw:
            x = F.pad(x, (0, pw, 0, ph))
        x = F.conv2d(x, self._w("embeddings.patch_embeddings.projection.weight"), self._w("embeddings.patch_embeddings.projection.bias"),
                     stride=cfg.patch)
        b, c, h, w = x.shape
        x = self._ln(x.flatten(2).transpose(1, 2), "embeddings.norm")
        out = []
        for s, depth in enumerate(cfg.depths):
            for i in range(depth):
                x = self._block(x, h, w, f"encoder.layers.{s}.blocks.{i}", cfg.heads[s], 0 if i % 2 == 0 else cfg.window // 2)
            if s + 1 in cfg.out_stages:
                y = self._ln(x, f"hidden_states_norms.stage{s + 1}")
                out.append(y.view(b, h, w, -1).permute(0, 3, 1, 2).contiguous())
            if s < len(cfg.depths) - 1:
                x = self._merge(x, h, w, f"encoder.layers.{s}.downsample")
                h, w = (h + 1) // 2, (w + 1) // 2
        return out
