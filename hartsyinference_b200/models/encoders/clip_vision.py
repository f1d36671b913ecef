"""CLIP vision transformer (ViT): non-overlapping patch embedding, class token, learned positions,
pre-LayerNorm, bidirectional pre-norm blocks with quick-GELU MLPs. Serves as the image embedder
(pooled class token after the post-LayerNorm) and as the vision tower of LLaVA-style models
(patch states of a chosen layer).

Reference: src/HartsyInference.Vision/ (CLIP / SigLIP embedders) and
src/HartsyInference.LLM/Multimodal/ (vision towers of the VLMs). Hugging Face ``CLIPVisionModel``
tensor names (``vision_model.*``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch

from ... import ops
from ..dit.common import WeightFactory


@dataclass(frozen=True)
class ClipVisionConfig:
    image_size: int = 336
    patch: int = 14
    width: int = 1024
    layers: int = 24
    heads: int = 16
    mlp_ratio: int = 4
    eps: float = 1e-5
    quick_gelu: bool = True

    @property
    def num_patches(self) -> int:
        return (self.image_size // self.patch) ** 2


def clip_vision_from_hf(d: dict) -> ClipVisionConfig:
    """Map the ``vision_config`` block of a Hugging Face CLIP / LLaVA ``config.json``."""
    return ClipVisionConfig(image_size=int(d.get("image_size", 224)), patch=int(d.get("patch_size", 14)),
                            width=int(d.get("hidden_size", 1024)), layers=int(d.get("num_hidden_layers", 24)),
                            heads=int(d.get("num_attention_heads", 16)),
                            mlp_ratio=int(d.get("intermediate_size", 4096)) // int(d.get("hidden_size", 1024)),
                            eps=float(d.get("layer_norm_eps", 1e-5)), quick_gelu=d.get("hidden_act", "quick_gelu") == "quick_gelu")


CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
CLIP_STD = (0.26862954, 0.26130258, 0.27577711)


def preprocess_image(image, size: int) -> torch.Tensor:
    """File path, PIL image, uint8 HWC array / tensor or float CHW tensor in [0, 1] -> normalised
    float [3, size, size]: bicubic resize of the short side to ``size``, centre crop, CLIP mean / std."""
    if isinstance(image, (str, bytes)) or hasattr(image, "__fspath__"):
        from PIL import Image
        image = Image.open(image)
    if hasattr(image, "convert"):       # PIL
        import numpy as np
        image = torch.from_numpy(np.asarray(image.convert("RGB")).copy())
    t = torch.as_tensor(image)
    if t.dtype == torch.uint8:
        t = t.float() / 255.0
    if t.ndim == 3 and t.shape[-1] == 3 and t.shape[0] != 3:
        t = t.permute(2, 0, 1)
    t = t.float()
    _, h, w = t.shape
    if (h, w) != (size, size):
        s = size / min(h, w)
        nh, nw = max(size, round(h * s)), max(size, round(w * s))
        t = torch.nn.functional.interpolate(t[None], size=(nh, nw), mode="bicubic", align_corners=False, antialias=True)[0]
        y0, x0 = (nh - size) // 2, (nw - size) // 2
        t = t[:, y0:y0 + size, x0:x0 + size].clamp(0, 1)
    mean = torch.tensor(CLIP_MEAN)[:, None, None]
    std = torch.tensor(CLIP_STD)[:, None, None]
    return (t - mean) / std


def tiny_clip_vision() -> ClipVisionConfig:
    return ClipVisionConfig(image_size=32, patch=8, width=128, layers=3, heads=2)


class ClipVisionEncoder:
    def __init__(self, cfg: ClipVisionConfig, device="cpu", get: Optional[Callable[[str], Optional[torch.Tensor]]] = None,
                 seed: int = 0, prefix: str = "vision_model.", pre_ln: str = "pre_layrnorm"):
        self.cfg, self.device = cfg, torch.device(device)
        f = WeightFactory(self.device, False, get=get, seed=seed)
        W, P = cfg.width, cfg.patch
        e = prefix + "embeddings."
        self.cls = f.tensor(e + "class_embedding", W)
        pw = f.tensor(e + "patch_embedding.weight", W, 3, P, P)
        # the patch GEMM's K (3 P P) is zero-padded to a multiple of 64 for the tensor-core tiles
        self.k_pad = -(-3 * P * P // 64) * 64
        w2 = torch.zeros(W, self.k_pad, dtype=pw.dtype, device=pw.device)
        w2[:, : 3 * P * P] = pw.reshape(W, 3 * P * P)
        self.patch = ops.LinearWeight(w2)
        self.pos = f.tensor(e + "position_embedding.weight", cfg.num_patches + 1, W)
        # (sic) CLIP checkpoints spell it "pre_layrnorm"; OWL-ViT's spell it out
        self.pre_w = f.tensor(prefix + pre_ln + ".weight", W, ones=True)
        self.pre_b = f.tensor(prefix + pre_ln + ".bias", W, zeros=True)
        self.blocks = []
        for i in range(cfg.layers):
            p = f"{prefix}encoder.layers.{i}."
            self.blocks.append(dict(
                ln1w=f.tensor(p + "layer_norm1.weight", W, ones=True), ln1b=f.tensor(p + "layer_norm1.bias", W, zeros=True),
                qkv=f.linear([p + f"self_attn.{n}_proj" for n in ("q", "k", "v")], [W, W, W], W),
                o=f.linear(p + "self_attn.out_proj", W, W),
                ln2w=f.tensor(p + "layer_norm2.weight", W, ones=True), ln2b=f.tensor(p + "layer_norm2.bias", W, zeros=True),
                fc1=f.linear(p + "mlp.fc1", cfg.mlp_ratio * W, W), fc2=f.linear(p + "mlp.fc2", W, cfg.mlp_ratio * W)))
        self.post_w = f.tensor(prefix + "post_layernorm.weight", W, ones=True)
        self.post_b = f.tensor(prefix + "post_layernorm.bias", W, zeros=True)

    def patchify(self, image: torch.Tensor) -> torch.Tensor:
        """image [3, H, W] (already normalised) -> [num_patches, k_pad]: (c, py, px) order, zero tail."""
        P = self.cfg.patch
        c, h, w = image.shape
        x = image.reshape(c, h // P, P, w // P, P).permute(1, 3, 0, 2, 4).reshape((h // P) * (w // P), c * P * P)
        return torch.nn.functional.pad(x, (0, self.k_pad - c * P * P))

    @torch.no_grad()
    def hidden_states(self, image: torch.Tensor, layer: int = -1) -> torch.Tensor:
        """[1 + num_patches, W] after block ``layer`` (negative counts from the end; -2 is what
        LLaVA feeds its projector). Row 0 is the class token."""
        cfg = self.cfg
        dt = torch.bfloat16
        patches = self.patchify(image.to(self.device).float()).to(dt)
        x = ops.linear(patches.contiguous(), self.patch)
        x = torch.cat([self.cls.to(dt)[None], x], 0)
        x = (x.float() + self.pos[: x.shape[0]].float()).to(dt)
        x, _, _ = ops.norm(x, self.pre_w, bias=self.pre_b, layernorm=True, eps=cfg.eps)
        L = x.shape[0]
        d = cfg.width // cfg.heads
        last = cfg.layers + layer + 1 if layer < 0 else layer
        for b in self.blocks[:last]:
            h, _, _ = ops.norm(x, b["ln1w"], bias=b["ln1b"], layernorm=True, eps=cfg.eps)
            q, k, v = ops.dit_qkv(ops.linear(h, b["qkv"]), cfg.heads, cfg.heads, d)
            a = ops.attention(q, k, v, causal=False)
            x = ops.linear(a.reshape(L, -1), b["o"], residual=x)
            h, _, _ = ops.norm(x, b["ln2w"], bias=b["ln2b"], layernorm=True, eps=cfg.eps)
            m = ops.linear(h, b["fc1"]).float()
            m = (m * torch.sigmoid(1.702 * m)) if cfg.quick_gelu else torch.nn.functional.gelu(m)
            x = ops.linear(m.to(dt), b["fc2"], residual=x)
        return x

    @torch.no_grad()
    def embed(self, image: torch.Tensor) -> torch.Tensor:
        """Pooled image feature: post-LayerNorm of the class token."""
        x = self.hidden_states(image)
        out, _, _ = ops.norm(x[:1].contiguous(), self.post_w, bias=self.post_b, layernorm=True, eps=self.cfg.eps)
        return out[0]
