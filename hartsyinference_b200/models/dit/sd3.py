"""Stable Diffusion 3 / 3.5 MMDiT transformer.

Latents are cut into 2 x 2 patches and embedded by a linear layer (the checkpoint's patch
convolution, flattened), plus a crop of a fixed 2-D sin-cos position table; text tokens go through
``context_embedder``. Every block keeps two streams (image, text) with their own AdaLN-Zero
modulation, projections and MLP, and one joint attention over [text | image] without rotary
embedding (SD3.5 adds per-head RMSNorm on q / k). The last block only reads the text stream (its
text side has no output projection or MLP). Output: AdaLN, projection to patch pixels, un-patchify.

The block math is the same set of fused ops the Flux double-stream block uses (AdaLN norm,
qkv split + head norm, gated residual, tensor-core GEMMs).

Reference: src/HartsyInference.Diffusion/Models/Denoisers/Sd3/, Pipelines/Sd3Pipeline.cs.
Tensor names follow diffusers ``SD3Transformer2DModel``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch

from ... import ops
from .common import WeightFactory, modulation, silu, timestep_embedding


@dataclass(frozen=True)
class Sd3Config:
    in_channels: int = 16
    patch: int = 2
    num_layers: int = 24
    num_heads: int = 24
    head_dim: int = 64
    context_dim: int = 4096
    pooled_dim: int = 2048
    pos_embed_max_size: int = 192
    qk_norm: bool = False            # SD3.5: RMSNorm on q and k heads
    mlp_ratio: float = 4.0

    @property
    def hidden_size(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def mlp_dim(self) -> int:
        return int(self.hidden_size * self.mlp_ratio)


SD3_MEDIUM = Sd3Config()
SD35_LARGE = Sd3Config(num_layers=38, num_heads=38, qk_norm=True)


def tiny_sd3(**over) -> Sd3Config:
    kw = dict(in_channels=4, num_layers=3, num_heads=2, head_dim=64, context_dim=64, pooled_dim=32, pos_embed_max_size=12)
    kw.update(over)
    return Sd3Config(**kw)


def sd3_from_hf(d: dict) -> Sd3Config:
    return Sd3Config(in_channels=d.get("in_channels", 16), patch=d.get("patch_size", 2), num_layers=d["num_layers"],
                     num_heads=d["num_attention_heads"], head_dim=d.get("attention_head_dim", 64),
                     context_dim=d.get("joint_attention_dim", 4096), pooled_dim=d.get("pooled_projection_dim", 2048),
                     pos_embed_max_size=d.get("pos_embed_max_size", 192), qk_norm=d.get("qk_norm") == "rms_norm")


def sincos_2d(dim: int, size: int) -> torch.Tensor:
    """[size * size, dim] table: half the channels encode the column, half the row (each half sin | cos)."""
    def axis(pos, d):
        omega = 1.0 / 10000 ** (torch.arange(d // 2, dtype=torch.float64) / (d / 2))
        out = pos.reshape(-1)[:, None] * omega[None]
        return torch.cat([out.sin(), out.cos()], 1)
    g = torch.arange(size, dtype=torch.float64)
    gy, gx = torch.meshgrid(g, g, indexing="ij")
    return torch.cat([axis(gx, dim // 2), axis(gy, dim // 2)], 1).float()


class Sd3Transformer:
    def __init__(self, cfg: Sd3Config = SD3_MEDIUM, device="cpu", fp8: bool = False,
                 get: Optional[Callable[[str], Optional[torch.Tensor]]] = None, seed: int = 0):
        self.cfg, self.device = cfg, torch.device(device)
        self.fp8 = fp8 and self.device.type == "cuda"
        f = WeightFactory(self.device, fp8, get=get, seed=seed)
        H, D, P, C = cfg.hidden_size, cfg.head_dim, cfg.patch, cfg.in_channels
        pw = f.tensor("pos_embed.proj.weight", H, C, P, P)
        self.x_embedder = ops.LinearWeight(pw.reshape(H, C * P * P).contiguous(), None, f.tensor("pos_embed.proj.bias", H, zeros=True))
        table = get("pos_embed.pos_embed") if get is not None else None
        n = cfg.pos_embed_max_size
        self.pos_table = (table.reshape(n, n, H) if table is not None else sincos_2d(H, n).reshape(n, n, H)).float().to(self.device)
        self.context_embedder = f.linear("context_embedder", H, cfg.context_dim)
        self.t_in = f.linear("time_text_embed.timestep_embedder.linear_1", H, 256, allow_fp8=False)
        self.t_out = f.linear("time_text_embed.timestep_embedder.linear_2", H, H)
        self.p_in = f.linear("time_text_embed.text_embedder.linear_1", H, cfg.pooled_dim, allow_fp8=False)
        self.p_out = f.linear("time_text_embed.text_embedder.linear_2", H, H)
        self.blocks = []
        for i in range(cfg.num_layers):
            p = f"transformer_blocks.{i}."
            last = i == cfg.num_layers - 1
            norm = (lambda n_: f.tensor(p + n_, D, ones=True)) if cfg.qk_norm else (lambda n_: None)
            b = dict(
                mod_i=f.linear(p + "norm1.linear", 6 * H, H),
                qkv_i=f.linear([p + "attn.to_q", p + "attn.to_k", p + "attn.to_v"], [H, H, H], H),
                qn_i=norm("attn.norm_q.weight"), kn_i=norm("attn.norm_k.weight"),
                out_i=f.linear(p + "attn.to_out.0", H, H),
                ff1_i=f.linear(p + "ff.net.0.proj", cfg.mlp_dim, H), ff2_i=f.linear(p + "ff.net.2", H, cfg.mlp_dim),
                mod_t=f.linear(p + "norm1_context.linear", (2 if last else 6) * H, H),
                qkv_t=f.linear([p + "attn.add_q_proj", p + "attn.add_k_proj", p + "attn.add_v_proj"], [H, H, H], H),
                qn_t=norm("attn.norm_added_q.weight"), kn_t=norm("attn.norm_added_k.weight"), last=last)
            if not last:
                b.update(out_t=f.linear(p + "attn.to_add_out", H, H),
                         ff1_t=f.linear(p + "ff_context.net.0.proj", cfg.mlp_dim, H), ff2_t=f.linear(p + "ff_context.net.2", H, cfg.mlp_dim))
            self.blocks.append(b)
        self.norm_out = f.linear("norm_out.linear", 2 * H, H)
        self.proj_out = f.linear("proj_out", P * P * C, H)

    def _pos(self, gh: int, gw: int) -> torch.Tensor:
        n = self.cfg.pos_embed_max_size
        top, left = (n - gh) // 2, (n - gw) // 2
        return self.pos_table[top:top + gh, left:left + gw].reshape(gh * gw, -1)

    def time_embedding(self, timestep: torch.Tensor, pooled: torch.Tensor) -> torch.Tensor:
        dt = torch.bfloat16
        te = timestep_embedding(timestep * 1000.0, 256).to(dt)
        temb = ops.linear(ops.linear(te, self.t_in, act="silu"), self.t_out).float()
        return (temb + ops.linear(ops.linear(pooled.to(dt), self.p_in, act="silu"), self.p_out).float()).to(dt)

    @torch.no_grad()
    def forward(self, latents: torch.Tensor, txt: torch.Tensor, timestep: torch.Tensor, pooled: torch.Tensor) -> torch.Tensor:
        """latents [1, C, h, w], txt [1, S_t, context_dim], timestep (sigma) [1], pooled [1, pooled_dim]
        -> velocity [1, C, h, w] (bf16)."""
        cfg = self.cfg
        H, D, P, C, nh = cfg.hidden_size, cfg.head_dim, cfg.patch, cfg.in_channels, cfg.num_heads
        dt = torch.bfloat16
        _, _, h, w = latents.shape
        gh, gw = h // P, w // P
        S_i, S_t = gh * gw, txt.shape[1]
        patches = latents.to(self.device).reshape(C, gh, P, gw, P).permute(1, 3, 0, 2, 4).reshape(S_i, C * P * P)
        x_i = (ops.linear(patches.to(dt).contiguous(), self.x_embedder).float() + self._pos(gh, gw)).to(dt)
        x_t = ops.linear(txt[0].to(self.device).to(dt).contiguous(), self.context_embedder)
        temb_act = silu(self.time_embedding(timestep.to(self.device), pooled.to(self.device)))

        def pre(x, mod, qkv_w, qn, kn, S):
            xn, _, _ = ops.norm(x, None, shift=mod[:, 0:H], scale=mod[:, H:2 * H], rows_per_batch=S, layernorm=True)
            return ops.dit_qkv(ops.linear(xn, qkv_w), nh, nh, D, q_norm_w=qn, k_norm_w=kn)

        def post(x, a, mod, out_w, ff1, ff2, S):
            x = ops.gated_residual(x, ops.linear(a, out_w), mod[:, 2 * H:3 * H], S)
            xn, _, _ = ops.norm(x, None, shift=mod[:, 3 * H:4 * H], scale=mod[:, 4 * H:5 * H], rows_per_batch=S, layernorm=True)
            return ops.gated_residual(x, ops.linear(ops.linear(xn, ff1, act="gelu_tanh"), ff2), mod[:, 5 * H:6 * H], S)

        for b in self.blocks:
            mod_i, mod_t = modulation(temb_act, b["mod_i"]), modulation(temb_act, b["mod_t"])
            if b["last"]:        # the text side of the last block is normalised with (scale, shift) only
                mod_t = torch.cat([mod_t[:, H:2 * H], mod_t[:, 0:H]], 1)
            qi, ki, vi = pre(x_i, mod_i, b["qkv_i"], b["qn_i"], b["kn_i"], S_i)
            qt, kt, vt = pre(x_t, mod_t, b["qkv_t"], b["qn_t"], b["kn_t"], S_t)
            att = ops.attention(torch.cat([qt, qi], 0), torch.cat([kt, ki], 0), torch.cat([vt, vi], 0)).reshape(S_t + S_i, H)
            x_i = post(x_i, att[S_t:].contiguous(), mod_i, b["out_i"], b["ff1_i"], b["ff2_i"], S_i)
            if not b["last"]:
                x_t = post(x_t, att[:S_t].contiguous(), mod_t, b["out_t"], b["ff1_t"], b["ff2_t"], S_t)
        mo = ops.linear(temb_act, self.norm_out)                               # [1, 2H]: scale, shift
        xn, _, _ = ops.norm(x_i.contiguous(), None, shift=mo[:, H:2 * H], scale=mo[:, 0:H], rows_per_batch=S_i, layernorm=True)
        out = ops.linear(xn, self.proj_out)                                    # [S_i, P * P * C], pixel-major inside a patch
        return out.reshape(gh, gw, P, P, C).permute(4, 0, 2, 1, 3).reshape(1, C, h, w)
