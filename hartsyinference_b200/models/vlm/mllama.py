"""Llama 3.2 Vision (Mllama): the tiled vision tower, its projector, and the glue that hands the
projected vision states to the decoder's cross-attention layers.

Tower: every image is up to ``max_tiles`` square tiles. Per tile: patch conv -> + gated per-tile
embedding (chosen by the aspect-ratio id) -> class token -> gated position + tile-position
embeddings -> LayerNorm -> patches padded to a multiple of 8 -> ``layers`` plain ViT blocks over
all tiles of the image at once -> LayerNorm -> post per-tile embedding -> ``global_layers`` gated
blocks. The output concatenates the final states with the states after the layers listed in
``intermediate`` ([tiles * (patches + 1), hidden * (1 + len(intermediate))]), and a linear projector
maps it to the decoder width. The attention mask only blocks padding-to-padding pairs (the model
was trained that way). Reference: src/HartsyInference.Core/Multimodal/ (Mllama).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.nn.functional as F


@dataclass(frozen=True)
class MllamaVisionConfig:
    hidden: int = 1280
    heads: int = 16
    ffn: int = 5120
    layers: int = 32
    global_layers: int = 8
    image_size: int = 560
    patch: int = 14
    max_tiles: int = 4
    eps: float = 1e-5
    intermediate: tuple = (3, 7, 15, 23, 30)
    supported_aspect_ratios: tuple = ((1, 1), (1, 2), (1, 3), (1, 4), (2, 1), (2, 2), (3, 1), (4, 1))

    @staticmethod
    def from_hf(d: dict) -> "MllamaVisionConfig":
        return MllamaVisionConfig(hidden=d.get("hidden_size", 1280), heads=d.get("attention_heads", 16),
                                  ffn=d.get("intermediate_size", 5120), layers=d.get("num_hidden_layers", 32),
                                  global_layers=d.get("num_global_layers", 8), image_size=d.get("image_size", 560),
                                  patch=d.get("patch_size", 14), max_tiles=d.get("max_num_tiles", 4),
                                  eps=d.get("norm_eps", 1e-5),
                                  intermediate=tuple(d.get("intermediate_layers_indices") or (3, 7, 15, 23, 30)),
                                  supported_aspect_ratios=tuple(tuple(a) for a in d.get("supported_aspect_ratios")
                                                                or MllamaVisionConfig.supported_aspect_ratios))


class _Block:
    def __init__(self, get: Callable, p: str, gated: bool, dev, dt):
        t = lambda n: get(p + n).to(dt).to(dev)
        self.q, self.k, self.v, self.o = (t(f"self_attn.{n}_proj.weight") for n in "qkvo")
        self.fc1_w, self.fc1_b, self.fc2_w, self.fc2_b = t("mlp.fc1.weight"), t("mlp.fc1.bias"), t("mlp.fc2.weight"), t("mlp.fc2.bias")
        self.n1_w, self.n1_b = t("input_layernorm.weight"), t("input_layernorm.bias")
        self.n2_w, self.n2_b = t("post_attention_layernorm.weight"), t("post_attention_layernorm.bias")
        self.g_attn = float(torch.tanh(get(p + "gate_attn").float()).reshape(-1)[0]) if gated else 1.0
        self.g_ffn = float(torch.tanh(get(p + "gate_ffn").float()).reshape(-1)[0]) if gated else 1.0

    def __call__(self, x: torch.Tensor, mask: torch.Tensor, heads: int, eps: float) -> torch.Tensor:
        n, c = x.shape
        d = c // heads
        h = F.layer_norm(x.float(), (c,), self.n1_w.float(), self.n1_b.float(), eps).to(x.dtype)
        q, k, v = (F.linear(h, w).reshape(n, heads, d).transpose(0, 1) for w in (self.q, self.k, self.v))
        a = F.scaled_dot_product_attention(q[None], k[None], v[None], attn_mask=mask.to(q.dtype))[0]
        x = x + self.g_attn * F.linear(a.transpose(0, 1).reshape(n, c), self.o)
        h = F.layer_norm(x.float(), (c,), self.n2_w.float(), self.n2_b.float(), eps).to(x.dtype)
        return x + self.g_ffn * F.linear(F.gelu(F.linear(h, self.fc1_w, self.fc1_b)), self.fc2_w, self.fc2_b)


class MllamaVisionTower:
    def __init__(self, cfg: MllamaVisionConfig, get: Callable[[str], Optional[torch.Tensor]], device="cpu",
                 dtype: torch.dtype = torch.bfloat16, prefix: str = "vision_model."):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype

        def t(n):
            w = get(prefix + n)
            if w is None:
                raise KeyError(f"missing tensor {prefix + n}")
            return w.to(dtype).to(self.device)

        self.patch_w = t("patch_embedding.weight")
        self.cls = t("class_embedding")
        self.pos, self.pos_tile = t("gated_positional_embedding.embedding"), t("gated_positional_embedding.tile_embedding.weight")
        self.pos_gate = float(torch.tanh(t("gated_positional_embedding.gate").float()).reshape(-1)[0])
        self.pre_tile = t("pre_tile_positional_embedding.embedding.weight")
        self.pre_gate = float(torch.tanh(t("pre_tile_positional_embedding.gate").float()).reshape(-1)[0])
        self.post_tile = t("post_tile_positional_embedding.embedding.weight")
        self.post_gate = float(torch.tanh(t("post_tile_positional_embedding.gate").float()).reshape(-1)[0])
        self.ln_pre = (t("layernorm_pre.weight"), t("layernorm_pre.bias"))
        self.ln_post = (t("layernorm_post.weight"), t("layernorm_post.bias"))
        g = lambda n: t(n)
        self.blocks = [_Block(lambda n: g(n), f"transformer.layers.{i}.", False, self.device, dtype) for i in range(cfg.layers)]
        self.global_blocks = [_Block(lambda n: g(n), f"global_transformer.layers.{i}.", True, self.device, dtype)
                              for i in range(cfg.global_layers)]

    @property
    def out_dim(self) -> int:
        return self.cfg.hidden * (1 + len(self.cfg.intermediate))

    def aspect_ratio_id(self, tiles_h: int, tiles_w: int) -> int:
        """1-based index into the supported (height, width) tile grids; 0 is the padding id."""
        return self.cfg.supported_aspect_ratios.index((tiles_h, tiles_w)) + 1

    @torch.no_grad()
    def __call__(self, tiles: torch.Tensor, aspect_ratio_id: int, num_tiles: Optional[int] = None) -> torch.Tensor:
        """tiles [max_tiles, 3, S, S] (unused tiles zero), the image's aspect-ratio id and how many
        tiles are real -> [max_tiles, patches + 1, hidden * (1 + len(intermediate))]."""
        cfg = self.cfg
        mt, c = cfg.max_tiles, cfg.hidden
        num_tiles = mt if num_tiles is None else num_tiles
        x = F.conv2d(tiles.to(self.device, self.dtype), self.patch_w, stride=cfg.patch).flatten(2).transpose(1, 2)   # [mt, P, C]
        p = x.shape[1] + 1
        x = x + self.pre_gate * self.pre_tile[aspect_ratio_id].reshape(mt, 1, c)
        x = torch.cat([self.cls.reshape(1, 1, c).expand(mt, 1, c), x], 1)
        x = x + (1 - self.pos_gate) * self.pos[None] + self.pos_gate * self.pos_tile[aspect_ratio_id].reshape(mt, p, c)
        x = F.layer_norm(x.float(), (c,), self.ln_pre[0].float(), self.ln_pre[1].float(), cfg.eps).to(self.dtype)
        pad = (8 - p % 8) % 8
        x = F.pad(x, (0, 0, 0, pad))
        pp = p + pad
        # 1 where a token is padding (an unused tile or a padded patch); only padding-to-padding pairs are blocked
        is_pad = torch.ones(mt, pp, device=self.device)
        is_pad[:num_tiles, :p] = 0
        is_pad = is_pad.reshape(-1)
        mask = (is_pad[:, None] * is_pad[None, :]) * torch.finfo(self.dtype).min
        x = x.reshape(mt * pp, c)
        taps = []
        for i, blk in enumerate(self.blocks):
            if i in cfg.intermediate:
                taps.append(x)
            x = blk(x, mask, cfg.heads, cfg.eps)
        x = F.layer_norm(x.float(), (c,), self.ln_post[0].float(), self.ln_post[1].float(), cfg.eps).to(self.dtype)
        x = (x.reshape(mt, pp, c) + self.post_gate * self.post_tile[aspect_ratio_id].reshape(mt, 1, c)).reshape(mt * pp, c)
        for blk in self.global_blocks:
            x = blk(x, mask, cfg.heads, cfg.eps)
        x = x.reshape(mt, pp, c)[:, :p]
        inter = torch.stack(taps, -1).reshape(mt, pp, c * len(taps))[:, :p]
        return torch.cat([x, inter], -1)


class MllamaModel:
    """Decoder + vision tower + projector. ``encode_image`` gives the cross-attention states of one
    image (real tiles only, so no cross-attention mask is needed); pass them to the decoder as
    ``ForwardBatch.cross_states`` for the prefill and for every decode step of that request."""

    def __init__(self, decoder, cfg: MllamaVisionConfig, get: Callable[[str], Optional[torch.Tensor]], image_token_id: int,
                 tower_prefix: str = "model.vision_model.", projector_prefix: str = "model.multi_modal_projector."):
        self.decoder, self.image_token_id = decoder, image_token_id
        dev = decoder.device
        self.tower = MllamaVisionTower(cfg, get, dev, torch.bfloat16, tower_prefix)
        self.proj_w = get(projector_prefix + "weight").to(torch.bfloat16).to(dev)
        self.proj_b = get(projector_prefix + "bias").to(torch.bfloat16).to(dev)

    @torch.no_grad()
    def encode_image(self, tiles: torch.Tensor, tiles_h: int, tiles_w: int) -> torch.Tensor:
        """tiles [max_tiles, 3, S, S] in row-major grid order (unused ones zero) -> [tiles_h * tiles_w * (patches + 1), hidden]."""
        n = tiles_h * tiles_w
        feats = self.tower(tiles, self.tower.aspect_ratio_id(tiles_h, tiles_w), n)[:n]
        out = F.linear(feats, self.proj_w, self.proj_b)
        return out.reshape(-1, out.shape[-1]).contiguous()

    def split_image(self, image: torch.Tensor) -> tuple[torch.Tensor, int, int]:
        """image [3, H, W] in [0, 1] -> (tiles, tiles_h, tiles_w): the supported tile grid closest to
        the image's aspect ratio, the image resized to fill it, CLIP-normalised."""
        from ..encoders.clip_vision import CLIP_MEAN, CLIP_STD
        cfg = self.tower.cfg
        _, h, w = image.shape
        grids = [g for g in cfg.supported_aspect_ratios if g[0] * g[1] <= cfg.max_tiles]
        th, tw = min(grids, key=lambda g: (abs(g[0] / g[1] - h / w), -g[0] * g[1]))
        s = cfg.image_size
        x = F.interpolate(image[None].float(), size=(th * s, tw * s), mode="bilinear", align_corners=False, antialias=True)[0]
        x = (x - torch.tensor(CLIP_MEAN).view(3, 1, 1)) / torch.tensor(CLIP_STD).view(3, 1, 1)
        tiles = torch.zeros(cfg.max_tiles, 3, s, s)
        tiles[:th * tw] = x.reshape(3, th, s, tw, s).permute(1, 3, 0, 2, 4).reshape(th * tw, 3, s, s)
        return tiles, th, tw
