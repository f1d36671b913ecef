"""CLIP text encoder (CLIP-L: 12 layers, width 768, 12 heads, causal mask, quick-GELU; pooled
output = final-LayerNorm state at the end-of-text token). Conditions Flux (pooled vector) and the SD
families. Reference: src/HartsyInference.Diffusion/Models/TextEncoders/ (CLIP-L / CLIP-G)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch

from ... import ops
from ..dit.common import WeightFactory


@dataclass(frozen=True)
class ClipTextConfig:
    vocab_size: int = 49408
    width: int = 768
    layers: int = 12
    heads: int = 12
    max_len: int = 77
    mlp_ratio: int = 4
    eps: float = 1e-5
    quick_gelu: bool = True


CLIP_L = ClipTextConfig()
# OpenCLIP bigG text tower (SDXL / SD3 second encoder): GELU, projection to 1280
CLIP_G = ClipTextConfig(width=1280, layers=32, heads=20, quick_gelu=False)


def clip_text_from_hf(d: dict) -> ClipTextConfig:
    width = d.get("hidden_size", 768)
    return ClipTextConfig(vocab_size=d.get("vocab_size", 49408), width=width, layers=d.get("num_hidden_layers", 12),
                          heads=d.get("num_attention_heads", 12), max_len=d.get("max_position_embeddings", 77),
                          mlp_ratio=d.get("intermediate_size", 4 * width) // width, eps=d.get("layer_norm_eps", 1e-5),
                          quick_gelu=d.get("hidden_act", "quick_gelu") == "quick_gelu")


def tiny_clip() -> ClipTextConfig:
    return ClipTextConfig(vocab_size=128, width=64, layers=2, heads=4, max_len=16)


class ClipTextEncoder:
    def __init__(self, cfg: ClipTextConfig = CLIP_L, device="cpu", get: Optional[Callable[[str], Optional[torch.Tensor]]] = None, seed: int = 0):
        self.cfg, self.device = cfg, torch.device(device)
        f = WeightFactory(self.device, False, get=get, seed=seed)
        W = cfg.width
        p0 = "text_model."
        self.tok = f.tensor(p0 + "embeddings.token_embedding.weight", cfg.vocab_size, W)
        self.pos = f.tensor(p0 + "embeddings.position_embedding.weight", cfg.max_len, W)
        self.blocks = []
        for i in range(cfg.layers):
            p = f"{p0}encoder.layers.{i}."
            q, k, v = (f.linear(p + f"self_attn.{n}_proj", W, W) for n in ("q", "k", "v"))
            self.blocks.append(dict(
                ln1w=f.tensor(p + "layer_norm1.weight", W, ones=True), ln1b=f.tensor(p + "layer_norm1.bias", W, zeros=True),
                qkv=ops.LinearWeight(torch.cat([q.weight, k.weight, v.weight], 0), None, torch.cat([q.bias, k.bias, v.bias], 0)),
                o=f.linear(p + "self_attn.out_proj", W, W),
                ln2w=f.tensor(p + "layer_norm2.weight", W, ones=True), ln2b=f.tensor(p + "layer_norm2.bias", W, zeros=True),
                fc1=f.linear(p + "mlp.fc1", cfg.mlp_ratio * W, W), fc2=f.linear(p + "mlp.fc2", W, cfg.mlp_ratio * W)))
        self.lnfw = f.tensor(p0 + "final_layer_norm.weight", W, ones=True)
        self.lnfb = f.tensor(p0 + "final_layer_norm.bias", W, zeros=True)
        # CLIPTextModelWithProjection checkpoints carry the projection of the pooled vector
        proj = get("text_projection.weight") if get is not None else None
        self.projection = None if proj is None else proj.float().to(self.device)

    @torch.no_grad()
    def encode(self, ids: torch.Tensor, layer: int = -1, project: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
        """ids [L] -> (hidden [L, W], pooled [W]); pooled is taken at the highest token id (end of text)
        after the final LayerNorm. ``layer`` = -2 returns the states after the second-to-last block
        without the final norm (what SDXL / SD3 condition on); ``project`` applies the checkpoint's
        text projection to the pooled vector."""
        cfg = self.cfg
        L = ids.shape[0]
        ids = ids.long().to(self.device)
        x = (self.tok[ids].float() + self.pos[:L].float()).to(torch.bfloat16)
        d = cfg.width // cfg.heads
        tapped = None
        stop = cfg.layers + layer + 1 if layer < 0 else layer
        for bi, b in enumerate(self.blocks):
            if bi == stop:
                tapped = x
            h, _, _ = ops.norm(x, b["ln1w"], bias=b["ln1b"], layernorm=True, eps=cfg.eps)
            qkv = ops.linear(h, b["qkv"])
            q, k, v = ops.dit_qkv(qkv, cfg.heads, cfg.heads, d)
            a = ops.attention(q, k, v, causal=True)
            x = ops.linear(a.reshape(L, -1), b["o"], residual=x)
            h, _, _ = ops.norm(x, b["ln2w"], bias=b["ln2b"], layernorm=True, eps=cfg.eps)
            m = ops.linear(h, b["fc1"]).float()
            m = (m * torch.sigmoid(1.702 * m)) if cfg.quick_gelu else torch.nn.functional.gelu(m)
            x = ops.linear(m.to(torch.bfloat16), b["fc2"], residual=x)
        out, _, _ = ops.norm(x, self.lnfw, bias=self.lnfb, layernorm=True, eps=cfg.eps)
        pooled = out[int(ids.argmax())]
        if project and self.projection is not None:
            pooled = (pooled.float() @ self.projection.t()).to(out.dtype)
        return (out if tapped is None else tapped), pooled
