"""SigLIP and DINOv2 vision transformers (image embedders and vision towers).

Both are pre-LayerNorm ViTs over non-overlapping patches. SigLIP has no class token and pools with
one learned query attending over the patch states followed by an MLP; DINOv2 prepends a class token,
scales each residual branch by a learned per-channel factor, and its embedding is the class token
(optionally concatenated with the mean patch token) after the final LayerNorm.

Reference: src/HartsyInference.Vision/Siglip/, src/HartsyInference.Vision/Dinov2/,
src/HartsyInference.LLM/Multimodal/ (SigLIP towers of the VLMs). Tensor names follow Hugging Face
``SiglipVisionModel`` (``vision_model.*``) and ``Dinov2Model``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch

from ... import ops
from ..dit.common import WeightFactory


@dataclass(frozen=True)
class VitConfig:
    kind: str = "siglip"          # siglip | dinov2 | vit (Hugging Face ViTModel names: DINO v1, the image tokenizer of TripoSR)
    image_size: int = 224
    patch: int = 16
    width: int = 768
    layers: int = 12
    heads: int = 12
    ffn: int = 3072
    eps: float = 1e-6
    activation: str = "gelu_tanh"  # gelu_tanh (SigLIP) | gelu (DINOv2)

    @property
    def num_patches(self) -> int:
        return (self.image_size // self.patch) ** 2


def tiny_vit(kind: str) -> VitConfig:
    return VitConfig(kind=kind, image_size=32, patch=8, width=128, layers=2, heads=2, ffn=256,
                     activation="gelu_tanh" if kind == "siglip" else "gelu")


def vit_from_hf(d: dict) -> VitConfig:
    kind = "dinov2" if d.get("model_type") == "dinov2" else "siglip"
    width = int(d["hidden_size"])
    ffn = int(d.get("intermediate_size") or width * int(d.get("mlp_ratio", 4)))
    act = d.get("hidden_act", "gelu")
    return VitConfig(kind=kind, image_size=int(d.get("image_size", 224)), patch=int(d.get("patch_size", 16)), width=width,
                     layers=int(d["num_hidden_layers"]), heads=int(d["num_attention_heads"]), ffn=ffn,
                     eps=float(d.get("layer_norm_eps", 1e-6)), activation="gelu_tanh" if "tanh" in act else "gelu")


def _act(x: torch.Tensor, name: str) -> torch.Tensor:
    return torch.nn.functional.gelu(x.float(), approximate="tanh" if name == "gelu_tanh" else "none").to(torch.bfloat16)


class VitEncoder:
    def __init__(self, cfg: VitConfig, device="cpu", get: Optional[Callable[[str], Optional[torch.Tensor]]] = None, seed: int = 0,
                 prefix: Optional[str] = None):
        self.cfg, self.device = cfg, torch.device(device)
        f = WeightFactory(self.device, False, get=get, seed=seed)
        W, P = cfg.width, cfg.patch
        sig = cfg.kind == "siglip"
        pre = prefix if prefix is not None else ("vision_model." if sig else "")
        names = dict(
            patch=pre + ("embeddings.patch_embedding" if sig else "embeddings.patch_embeddings.projection"),
            pos=pre + ("embeddings.position_embedding.weight" if sig else "embeddings.position_embeddings"),
            layer=pre + ("encoder.layers.{}." if sig else "encoder.layer.{}."),
            final=pre + ("post_layernorm" if sig else "layernorm"))
        pw = f.tensor(names["patch"] + ".weight", W, 3, P, P)
        self.k_pad = -(-3 * P * P // 64) * 64          # patch GEMM K zero-padded to the tensor-core tile
        w2 = torch.zeros(W, self.k_pad, dtype=pw.dtype, device=pw.device)
        w2[:, : 3 * P * P] = pw.reshape(W, 3 * P * P)
        self.patch = ops.LinearWeight(w2, None, f.tensor(names["patch"] + ".bias", W, zeros=True))
        n_pos = cfg.num_patches + (0 if sig else 1)
        self.pos = f.tensor(names["pos"], n_pos, W).reshape(n_pos, W)
        self.cls = None if sig else f.tensor(pre + "embeddings.cls_token", W).reshape(W)
        self.blocks = []
        for i in range(cfg.layers):
            p = names["layer"].format(i)
            if sig:
                qkv = [p + f"self_attn.{n}_proj" for n in ("q", "k", "v")]
                o, n1, n2, fc1, fc2 = p + "self_attn.out_proj", p + "layer_norm1", p + "layer_norm2", p + "mlp.fc1", p + "mlp.fc2"
            elif cfg.kind == "vit":
                qkv = [p + f"attention.attention.{n}" for n in ("query", "key", "value")]
                o, n1, n2 = p + "attention.output.dense", p + "layernorm_before", p + "layernorm_after"
                fc1, fc2 = p + "intermediate.dense", p + "output.dense"
            else:
                qkv = [p + f"attention.attention.{n}" for n in ("query", "key", "value")]
                o, n1, n2, fc1, fc2 = p + "attention.output.dense", p + "norm1", p + "norm2", p + "mlp.fc1", p + "mlp.fc2"
            b = dict(qkv=f.linear(qkv, [W, W, W], W), o=f.linear(o, W, W),
                     n1=(f.tensor(n1 + ".weight", W, ones=True), f.tensor(n1 + ".bias", W, zeros=True)),
                     n2=(f.tensor(n2 + ".weight", W, ones=True), f.tensor(n2 + ".bias", W, zeros=True)),
                     fc1=f.linear(fc1, cfg.ffn, W), fc2=f.linear(fc2, W, cfg.ffn))
            if cfg.kind == "dinov2":
                b["ls1"] = f.tensor(p + "layer_scale1.lambda1", W, ones=True)
                b["ls2"] = f.tensor(p + "layer_scale2.lambda1", W, ones=True)
            self.blocks.append(b)
        self.final = (f.tensor(names["final"] + ".weight", W, ones=True), f.tensor(names["final"] + ".bias", W, zeros=True))
        self.head = None
        if sig and (get is None or get(pre + "head.probe") is not None):
            h = pre + "head."
            ipw = f.tensor(h + "attention.in_proj_weight", 3 * W, W)
            ipb = f.tensor(h + "attention.in_proj_bias", 3 * W, zeros=True)
            self.head = dict(probe=f.tensor(h + "probe", W).reshape(1, W),
                             q=ops.LinearWeight(ipw[:W].contiguous(), None, ipb[:W].contiguous()),
                             kv=ops.LinearWeight(ipw[W:].contiguous(), None, ipb[W:].contiguous()),
                             o=f.linear(h + "attention.out_proj", W, W),
                             ln=(f.tensor(h + "layernorm.weight", W, ones=True), f.tensor(h + "layernorm.bias", W, zeros=True)),
                             fc1=f.linear(h + "mlp.fc1", cfg.ffn, W), fc2=f.linear(h + "mlp.fc2", W, cfg.ffn))

    def _ln(self, x, wb):
        return ops.norm(x, wb[0], bias=wb[1], layernorm=True, eps=self.cfg.eps)[0]

    def _patchify(self, image: torch.Tensor) -> torch.Tensor:
        P = self.cfg.patch
        c, h, w = image.shape
        x = image.reshape(c, h // P, P, w // P, P).permute(1, 3, 0, 2, 4).reshape((h // P) * (w // P), c * P * P)
        return torch.nn.functional.pad(x, (0, self.k_pad - c * P * P))

    def _positions(self, gh: int, gw: int) -> torch.Tensor:
        """Position table for a gh x gw patch grid: the stored one, or (for another image size) its
        patch part resampled bicubically, the class position kept."""
        n0 = int(round(self.cfg.num_patches ** 0.5))
        if (gh, gw) == (n0, n0):
            return self.pos
        extra = 0 if self.cls is None else 1
        grid = self.pos[extra:].float().reshape(1, n0, n0, -1).permute(0, 3, 1, 2)
        grid = torch.nn.functional.interpolate(grid, size=(gh, gw), mode="bicubic", align_corners=False)
        grid = grid.permute(0, 2, 3, 1).reshape(gh * gw, -1).to(self.pos.dtype)
        return torch.cat([self.pos[:extra], grid], 0)

    @torch.no_grad()
    def hidden_states(self, image: torch.Tensor, layer: int = -1, final_norm: bool = True, taps: Optional[list] = None):
        """image [3, H, W] normalised -> token states [(1 +) num_patches, W] after block ``layer``.
        With ``taps`` (1-based block counts) returns the final-normed states after each of those
        blocks instead (what dense-prediction heads consume)."""
        cfg, dt = self.cfg, torch.bfloat16
        x = ops.linear(self._patchify(image.to(self.device).float()).to(dt).contiguous(), self.patch)
        if self.cls is not None:
            x = torch.cat([self.cls.to(dt)[None], x], 0)
        pos = self._positions(image.shape[-2] // cfg.patch, image.shape[-1] // cfg.patch)
        x = (x.float() + pos[: x.shape[0]].float()).to(dt)
        L, d = x.shape[0], cfg.width // cfg.heads
        last = cfg.layers + layer + 1 if layer < 0 else layer
        if taps:
            last = max(taps)
        tapped = []
        for bi, b in enumerate(self.blocks[:last]):
            q, k, v = ops.dit_qkv(ops.linear(self._ln(x, b["n1"]), b["qkv"]), cfg.heads, cfg.heads, d)
            a = ops.linear(ops.attention(q, k, v, causal=False).reshape(L, -1), b["o"])
            if "ls1" in b:
                a = (a.float() * b["ls1"].float()).to(dt)
            x = (x.float() + a.float()).to(dt)
            m = ops.linear(_act(ops.linear(self._ln(x, b["n2"]), b["fc1"]), cfg.activation), b["fc2"])
            if "ls2" in b:
                m = (m.float() * b["ls2"].float()).to(dt)
            x = (x.float() + m.float()).to(dt)
            if taps and bi + 1 in taps:
                tapped.append(self._ln(x, self.final))
        if taps:
            return tapped
        return self._ln(x, self.final) if (final_norm and last == cfg.layers) else x

    @torch.no_grad()
    def embed(self, image: torch.Tensor, concat_patch_mean: bool = False) -> torch.Tensor:
        """Pooled image feature [W] (DINOv2 with ``concat_patch_mean``: [2 W])."""
        cfg = self.cfg
        x = self.hidden_states(image)
        if cfg.kind == "dinov2":
            return torch.cat([x[0], x[1:].float().mean(0).to(x.dtype)]) if concat_patch_mean else x[0]
        if self.head is None:
            return x.float().mean(0).to(x.dtype)
        h, d = self.head, cfg.width // cfg.heads
        q = ops.linear(h["probe"].to(torch.bfloat16), h["q"]).reshape(1, cfg.heads, d)
        kv = ops.linear(x, h["kv"]).reshape(x.shape[0], 2, cfg.heads, d)
        a = ops.attention(q, kv[:, 0].contiguous(), kv[:, 1].contiguous(), causal=False).reshape(1, -1)
        y = ops.linear(a, h["o"])
        m = ops.linear(_act(ops.linear(self._ln(y, h["ln"]), h["fc1"]), cfg.activation), h["fc2"])
        return (y.float() + m.float()).to(torch.bfloat16)[0]
