"""HuBERT / wav2vec 2.0 speech encoder: waveform -> content features at 50 Hz (the content encoder of voice
conversion and of speech-token front ends).

* feature encoder: seven 1-d convolutions (kernels 10, 3, 3, 3, 3, 2, 2; strides 5, 2, 2, 2, 2, 2, 2; total
  stride 320) with GELU; either one GroupNorm after the first convolution (base models) or a LayerNorm over
  channels after every convolution (large models);
* projection: LayerNorm over the 512 channels, Linear to the model width;
* positions: a grouped convolution (kernel 128, 16 groups, weight-normalised, the last output frame dropped
  because the kernel is even) + GELU, added to the input;
* transformer: post-LayerNorm blocks with a LayerNorm before the first (base) or pre-LayerNorm blocks with a
  final LayerNorm (``do_stable_layer_norm``, large models). ``hidden_states(layer)`` returns an intermediate
  layer, which is what downstream models consume (layer 9 or 12 for voice conversion).

Weights by the names of the `transformers` checkpoints (``hubert.*`` / ``wav2vec2.*`` prefixes are stripped).
Reference: src/HartsyInference.Audio/Models/Hubert/ (Hubert.cs, HubertConfig.cs).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.nn.functional as F


@dataclass(frozen=True)
class HubertConfig:
    hidden: int = 768
    layers: int = 12
    heads: int = 12
    ffn: int = 3072
    conv_dim: tuple = (512,) * 7
    conv_kernel: tuple = (10, 3, 3, 3, 3, 2, 2)
    conv_stride: tuple = (5, 2, 2, 2, 2, 2, 2)
    conv_bias: bool = False
    group_norm: bool = True              # False: LayerNorm after every convolution
    pos_kernel: int = 128
    pos_groups: int = 16
    stable_layer_norm: bool = False
    feat_proj_layer_norm: bool = True
    eps: float = 1e-5
    normalize_input: bool = False        # large models: zero-mean unit-variance waveform

    @staticmethod
    def from_hf(d: dict) -> "HubertConfig":
        return HubertConfig(hidden=d.get("hidden_size", 768), layers=d.get("num_hidden_layers", 12), heads=d.get("num_attention_heads", 12),
                            ffn=d.get("intermediate_size", 3072), conv_dim=tuple(d.get("conv_dim", (512,) * 7)),
                            conv_kernel=tuple(d.get("conv_kernel", (10, 3, 3, 3, 3, 2, 2))), conv_stride=tuple(d.get("conv_stride", (5, 2, 2, 2, 2, 2, 2))),
                            conv_bias=bool(d.get("conv_bias", False)), group_norm=d.get("feat_extract_norm", "group") == "group",
                            pos_kernel=d.get("num_conv_pos_embeddings", 128), pos_groups=d.get("num_conv_pos_embedding_groups", 16),
                            stable_layer_norm=bool(d.get("do_stable_layer_norm", False)),
                            feat_proj_layer_norm=bool(d.get("feat_proj_layer_norm", True)), eps=d.get("layer_norm_eps", 1e-5),
                            normalize_input=d.get("feat_extract_norm", "group") == "layer")


class Hubert:
    def __init__(self, cfg: HubertConfig, get: Callable[[str], Optional[torch.Tensor]], device="cpu", dtype: torch.dtype = torch.float32):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype

        def raw(n):
            for prefix in ("", "hubert.", "wav2vec2."):
                w = get(prefix + n)
                if w is not None:
                    return w
            return None

        def t(n, optional=False):
            w = raw(n)
            if w is None:
                if optional:
                    return None
                raise KeyError(n)
            return w.to(self.device).to(dtype)

        self.convs = []
        for i in range(len(cfg.conv_dim)):
            p = f"feature_extractor.conv_layers.{i}."
            self.convs.append({"w": t(p + "conv.weight"), "b": t(p + "conv.bias", True),
                               "norm": (t(p + "layer_norm.weight", True), t(p + "layer_norm.bias", True))})
        self.proj_norm = (t("feature_projection.layer_norm.weight", True), t("feature_projection.layer_norm.bias", True))
        self.proj = (t("feature_projection.projection.weight"), t("feature_projection.projection.bias"))
        # weight-normalised positional convolution: g * v / |v|, the norm taken over all but the kernel axis
        g = raw("encoder.pos_conv_embed.conv.parametrizations.weight.original0")
        v = raw("encoder.pos_conv_embed.conv.parametrizations.weight.original1")
        if g is None:
            g, v = raw("encoder.pos_conv_embed.conv.weight_g"), raw("encoder.pos_conv_embed.conv.weight_v")
        if g is not None:
            v = v.float()
            w = g.float() * v / v.norm(dim=(0, 1), keepdim=True)
        else:
            w = raw("encoder.pos_conv_embed.conv.weight").float()
        self.pos = (w.to(self.device).to(dtype), t("encoder.pos_conv_embed.conv.bias"))
        self.enc_norm = (t("encoder.layer_norm.weight"), t("encoder.layer_norm.bias"))
        self.blocks = []
        for i in range(cfg.layers):
            p = f"encoder.layers.{i}."
            lin = lambda n: (t(p + n + ".weight"), t(p + n + ".bias"))
            qkv = [lin(f"attention.{n}_proj") for n in "qkv"]
            self.blocks.append({"qkv": (torch.cat([w for w, _ in qkv], 0), torch.cat([b for _, b in qkv], 0)),
                                "out": lin("attention.out_proj"), "ln1": lin("layer_norm"),
                                "up": lin("feed_forward.intermediate_dense"), "down": lin("feed_forward.output_dense"),
                                "ln2": lin("final_layer_norm")})

    def frames(self, samples: int) -> int:
        n = samples
        for k, s in zip(self.cfg.conv_kernel, self.cfg.conv_stride):
            n = (n - k) // s + 1
        return n

    @torch.no_grad()
    def features(self, wave: torch.Tensor) -> torch.Tensor:
        """wave [B, samples] (16 kHz) -> convolutional features [B, frames, conv_dim]."""
        cfg = self.cfg
        x = wave.to(self.device).float()
        if x.dim() == 1:
            x = x[None]
        if cfg.normalize_input:
            x = (x - x.mean(-1, keepdim=True)) / torch.sqrt(x.var(-1, keepdim=True, unbiased=False) + 1e-7)
        x = x.to(self.dtype)[:, None]
        for i, c in enumerate(self.convs):
            x = F.conv1d(x, c["w"], c["b"], stride=cfg.conv_stride[i])
            if cfg.group_norm and i == 0:
                x = F.group_norm(x, x.shape[1], *c["norm"], eps=1e-5)
            elif not cfg.group_norm:
                x = F.layer_norm(x.transpose(1, 2), (x.shape[1],), *c["norm"], eps=1e-5).transpose(1, 2)
            x = F.gelu(x)
        return x.transpose(1, 2)

    @torch.no_grad()
    def all_hidden_states(self, wave: torch.Tensor) -> list:
        """The input of the first block and the output of every block (the last one with the closing norm where the
        model has one): ``layers + 1`` tensors [B, frames, hidden]. Codecs average these into a semantic feature."""
        return [self.hidden_states(wave, layer=i) for i in range(self.cfg.layers)] + [self.hidden_states(wave)]

    @torch.no_grad()
    def hidden_states(self, wave: torch.Tensor, layer: Optional[int] = None) -> torch.Tensor:
        """-> [B, frames, hidden] after ``layer`` transformer blocks (all of them, with the closing norm, when None)."""
        cfg = self.cfg
        x = self.features(wave)
        if cfg.feat_proj_layer_norm and self.proj_norm[0] is not None:
            x = F.layer_norm(x, (x.shape[-1],), *self.proj_norm, eps=cfg.eps)
        x = F.linear(x, *self.proj)
        pos = F.conv1d(x.transpose(1, 2), *self.pos, padding=cfg.pos_kernel // 2, groups=cfg.pos_groups)
        if cfg.pos_kernel % 2 == 0:
            pos = pos[:, :, :-1]
        x = x + F.gelu(pos).transpose(1, 2)
        h, hd = cfg.hidden, cfg.hidden // cfg.heads
        if not cfg.stable_layer_norm:
            x = F.layer_norm(x, (h,), *self.enc_norm, eps=cfg.eps)
        n = cfg.layers if layer is None else layer
        b, t, _ = x.shape
        for blk in self.blocks[:n]:
            y = F.layer_norm(x, (h,), *blk["ln1"], eps=cfg.eps) if cfg.stable_layer_norm else x
            q, k, v = F.linear(y, *blk["qkv"]).view(b, t, 3, cfg.heads, hd).permute(2, 0, 3, 1, 4)
            a = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(b, t, h)
            x = x + F.linear(a, *blk["out"])
            if cfg.stable_layer_norm:
                x = x + F.linear(F.gelu(F.linear(F.layer_norm(x, (h,), *blk["ln2"], eps=cfg.eps), *blk["up"])), *blk["down"])
            else:
                x = F.layer_norm(x, (h,), *blk["ln1"], eps=cfg.eps)
                x = F.layer_norm(x + F.linear(F.gelu(F.linear(x, *blk["up"])), *blk["down"]), (h,), *blk["ln2"], eps=cfg.eps)
        if cfg.stable_layer_norm and layer is None:
            x = F.layer_norm(x, (h,), *self.enc_norm, eps=cfg.eps)
        return x

    __call__ = hidden_states
