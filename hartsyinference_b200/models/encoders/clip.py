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

    @torch.no_grad()
    def encode(self, ids: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """ids [L] -> (hidden [L, W], pooled [W]); pooled is taken at the highest token id (end of text)."""
        cfg = self.cfg
        L = ids.shape[0]
        ids = ids.long().to(self.device)
        x = (self.tok[ids].float() + self.pos[:L].float()).to(torch.bfloat16)
        d = cfg.width // cfg.heads
        for b in self.blocks:
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
        return out, out[int(ids.argmax())]
