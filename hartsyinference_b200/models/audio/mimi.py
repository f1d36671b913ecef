"""Mimi: the 12.5 Hz streaming speech codec behind Moshi, the Kyutai speech-to-text / text-to-speech
models and CSM. 24 kHz mono -> 32 codebooks of 2048 entries per 80 ms frame, and back.

encode: causal SEANet encoder (7-tap convolution, four stages of [residual block, ELU, strided
convolution with kernel 2 x stride] at strides 4, 5, 6, 8, ELU, 3-tap convolution to 512 channels;
every convolution left-padded by kernel - stride, plus whatever right padding completes the last
frame) -> 8-layer causal transformer (RoPE, sliding window of 250 frames, LayerNorm, GELU MLP,
learned per-channel scales on both residual branches) -> stride-2 convolution to 12.5 Hz
(replicate padding) -> split residual vector quantiser: codebook 0 (semantic) quantises the
projected latent on its own, codebooks 1..31 (acoustic) quantise it again as a residual chain;
each group has its own 512 -> 256 input and 256 -> 512 output projection.

decode: sum of the two groups' outputs -> depthwise transposed convolution back to 25 Hz -> the
second 8-layer transformer -> SEANet decoder (mirror of the encoder, transposed convolutions
trimmed on the right).

Weights by the names of the `transformers` checkpoint (``kyutai/mimi``; an optional
``codec_model.`` / ``audio_encoder.`` prefix is given by the host model). Codebook tables are
stored as ``embed_sum`` / ``cluster_usage`` and divided at load.
Reference: src/HartsyInference.Audio/Models/Codecs/ (Mimi codec) and its users under
Models/Kyutai/, Models/Csm/.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.nn.functional as F


@dataclass(frozen=True)
class MimiConfig:
    hidden: int = 512
    filters: int = 64
    ratios: tuple = (8, 6, 5, 4)
    kernel: int = 7
    last_kernel: int = 3
    residual_kernel: int = 3
    residual_layers: int = 1
    dilation_growth: int = 2
    compress: int = 2
    conv_shortcut: bool = False
    pad_mode: str = "constant"
    codebook_size: int = 2048
    codebook_dim: int = 256
    quantizers: int = 32
    semantic_quantizers: int = 1
    layers: int = 8
    heads: int = 8
    kv_heads: int = 8
    head_dim: int = 64
    ffn: int = 2048
    window: int = 250
    rope_theta: float = 10000.0
    eps: float = 1e-5
    sampling_rate: int = 24000
    frame_rate: float = 12.5
    upsample_groups: int = 512

    @staticmethod
    def from_hf(d: dict) -> "MimiConfig":
        if not d.get("use_causal_conv", True):
            raise ValueError("only the causal (streaming) Mimi layout is supported")
        rope = d.get("rope_parameters") or {}
        hidden, heads = d.get("hidden_size", 512), d.get("num_attention_heads", 8)
        return MimiConfig(hidden=hidden, filters=d.get("num_filters", 64), ratios=tuple(d.get("upsampling_ratios") or (8, 6, 5, 4)),
                          kernel=d.get("kernel_size", 7), last_kernel=d.get("last_kernel_size", 3), residual_kernel=d.get("residual_kernel_size", 3),
                          residual_layers=d.get("num_residual_layers", 1), dilation_growth=d.get("dilation_growth_rate", 2),
                          compress=d.get("compress", 2), conv_shortcut=bool(d.get("use_conv_shortcut", False)), pad_mode=d.get("pad_mode", "constant"),
                          codebook_size=d.get("codebook_size", 2048), codebook_dim=d.get("codebook_dim", 256),
                          quantizers=d.get("num_quantizers", 32), semantic_quantizers=d.get("num_semantic_quantizers", 1),
                          layers=d.get("num_hidden_layers", 8), heads=heads, kv_heads=d.get("num_key_value_heads", heads),
                          head_dim=d.get("head_dim") or hidden // heads, ffn=d.get("intermediate_size", 2048), window=d.get("sliding_window", 250),
                          rope_theta=float(rope.get("rope_theta", d.get("rope_theta", 10000.0))), eps=d.get("norm_eps", 1e-5),
                          sampling_rate=d.get("sampling_rate", 24000), frame_rate=float(d.get("frame_rate") or d.get("_frame_rate") or 12.5),
                          upsample_groups=d.get("upsample_groups", hidden))

    @property
    def samples_per_frame(self) -> int:
        return int(round(self.sampling_rate / self.frame_rate))


class Mimi:
    def __init__(self, cfg: MimiConfig, get: Callable[[str], Optional[torch.Tensor]], device="cpu", dtype: torch.dtype = torch.float32,
                 prefix: str = ""):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        self._get, self._prefix, self._cache = get, prefix, {}
        self._books = {}

    # ------------------------------------------------------------------------------ weights
    def _w(self, name: str, optional: bool = False):
        hit = self._cache.get(name, False)
        if hit is False:
            w = self._get(self._prefix + name)
            if w is None and not optional:
                raise KeyError(self._prefix + name)
            hit = None if w is None else w.to(self.device).to(self.dtype)
            self._cache[name] = hit
        return hit

    def _book(self, group: str, i: int) -> torch.Tensor:
        key = (group, i)
        if key not in self._books:
            p = f"quantizer.{group}_residual_vector_quantizer.layers.{i}.codebook."
            self._books[key] = (self._w(p + "embed_sum").float() / self._w(p + "cluster_usage").float().clamp_min(1e-5)[:, None])
        return self._books[key]

    # ------------------------------------------------------------------------------ convolutions
    def _conv(self, x, p: str, stride: int = 1, dilation: int = 1, pad_mode: Optional[str] = None, groups: int = 1):
        w, b = self._w(p + ".conv.weight"), self._w(p + ".conv.bias", True)
        k_eff = (w.shape[-1] - 1) * dilation + 1
        total = k_eff - stride
        n = x.shape[-1]
        frames = math.ceil((n - k_eff + total) / stride + 1) - 1
        extra = frames * stride + k_eff - total - n
        mode = pad_mode or self.cfg.pad_mode
        x = F.pad(x, (total, extra), mode=mode) if (total or extra) else x
        return F.conv1d(x, w, b, stride=stride, dilation=dilation, groups=groups)

    def _conv_t(self, x, p: str, stride: int, groups: int = 1):
        w, b = self._w(p + ".conv.weight"), self._w(p + ".conv.bias", True)
        y = F.conv_transpose1d(x, w, b, stride=stride, groups=groups)
        trim = w.shape[-1] - stride
        return y[..., :y.shape[-1] - trim] if trim else y

    def _resblock(self, x, p: str, dilation: int):
        y = self._conv(F.elu(x), p + ".block.1", dilation=dilation)
        y = self._conv(F.elu(y), p + ".block.3")
        return (self._conv(x, p + ".shortcut") if self.cfg.conv_shortcut else x) + y

    # ------------------------------------------------------------------------------ transformer
    def _transformer(self, x: torch.Tensor, p: str) -> torch.Tensor:
        """x [B, T, H]; causal attention inside a window of ``cfg.window`` frames."""
        cfg = self.cfg
        b, t, h = x.shape
        pos = torch.arange(t, device=x.device)
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2, device=x.device).float() / cfg.head_dim))
        ang = pos[:, None].float() * inv[None]
        cos, sin = torch.cat([ang.cos(), ang.cos()], -1).to(x.dtype), torch.cat([ang.sin(), ang.sin()], -1).to(x.dtype)
        rot = lambda u: u * cos + torch.cat([-u[..., cfg.head_dim // 2:], u[..., :cfg.head_dim // 2]], -1) * sin
        delta = pos[:, None] - pos[None, :]
        mask = (delta >= 0) & (delta < cfg.window)
        for i in range(cfg.layers):
            q_ = f"{p}.layers.{i}."
            y = F.layer_norm(x, (h,), self._w(q_ + "input_layernorm.weight"), self._w(q_ + "input_layernorm.bias"), cfg.eps)
            lin = lambda n: F.linear(y, self._w(q_ + f"self_attn.{n}_proj.weight"), self._w(q_ + f"self_attn.{n}_proj.bias", True))
            q = rot(lin("q").view(b, t, cfg.heads, cfg.head_dim).transpose(1, 2))
            k = rot(lin("k").view(b, t, cfg.kv_heads, cfg.head_dim).transpose(1, 2))
            v = lin("v").view(b, t, cfg.kv_heads, cfg.head_dim).transpose(1, 2)
            a = F.scaled_dot_product_attention(q, k, v, attn_mask=mask, enable_gqa=cfg.kv_heads != cfg.heads)
            a = F.linear(a.transpose(1, 2).reshape(b, t, -1), self._w(q_ + "self_attn.o_proj.weight"), self._w(q_ + "self_attn.o_proj.bias", True))
            x = x + self._w(q_ + "self_attn_layer_scale.scale") * a
            y = F.layer_norm(x, (h,), self._w(q_ + "post_attention_layernorm.weight"), self._w(q_ + "post_attention_layernorm.bias"), cfg.eps)
            y = F.linear(F.gelu(F.linear(y, self._w(q_ + "mlp.fc1.weight"))), self._w(q_ + "mlp.fc2.weight"))
            x = x + self._w(q_ + "mlp_layer_scale.scale") * y
        return x

    # ------------------------------------------------------------------------------ quantiser
    def _group(self, i: int) -> tuple[str, int]:
        s = self.cfg.semantic_quantizers
        return ("semantic", i) if i < s else ("acoustic", i - s)

    @torch.no_grad()
    def quantize(self, z: torch.Tensor, quantizers: Optional[int] = None) -> torch.Tensor:
        """latents [B, hidden, frames] -> codes [B, n, frames]."""
        n = quantizers or self.cfg.quantizers
        s = self.cfg.semantic_quantizers
        out = []
        for group, count in (("semantic", min(n, s)), ("acoustic", max(n - s, 0))):
            if count == 0:
                continue
            proj = self._w(f"quantizer.{group}_residual_vector_quantizer.input_proj.weight", True)
            r = (F.conv1d(z, proj) if proj is not None else z).float().transpose(1, 2)
            for i in range(count):
                book = self._book(group, i)
                idx = torch.cdist(r, book[None].expand(r.shape[0], -1, -1)).argmin(-1)
                r = r - book[idx]
                out.append(idx)
        return torch.stack(out, 1)

    @torch.no_grad()
    def dequantize(self, codes: torch.Tensor) -> torch.Tensor:
        """codes [B, n, frames] -> latents [B, hidden, frames]."""
        # ids outside the tables (a language model's control ids) are clamped, never used as gather indices
        codes = codes.to(self.device).long().clamp(0, self.cfg.codebook_size - 1)
        s = self.cfg.semantic_quantizers
        total = None
        for group, lo, hi in (("semantic", 0, min(s, codes.shape[1])), ("acoustic", s, codes.shape[1])):
            if hi <= lo:
                continue
            q = sum(self._book(group, i - lo)[codes[:, i]] for i in range(lo, hi)).transpose(1, 2).to(self.dtype)
            proj = self._w(f"quantizer.{group}_residual_vector_quantizer.output_proj.weight", True)
            q = F.conv1d(q, proj) if proj is not None else q
            total = q if total is None else total + q
        return total

    # ------------------------------------------------------------------------------ public
    @torch.no_grad()
    def encode_latents(self, wave: torch.Tensor) -> torch.Tensor:
        """wave [B, 1, samples] or [B, samples] -> latents before quantisation [B, hidden, frames] at the frame rate."""
        cfg = self.cfg
        x = wave.to(self.device).to(self.dtype)
        if x.dim() == 2:
            x = x[:, None]
        x = self._conv(x, "encoder.layers.0")
        idx = 1
        for ratio in reversed(cfg.ratios):
            for j in range(cfg.residual_layers):
                x = self._resblock(x, f"encoder.layers.{idx}", cfg.dilation_growth ** j)
                idx += 1
            x = self._conv(F.elu(x), f"encoder.layers.{idx + 1}", stride=ratio)
            idx += 2
        x = self._conv(F.elu(x), f"encoder.layers.{idx + 1}")
        x = self._transformer(x.transpose(1, 2), "encoder_transformer").transpose(1, 2)
        if self._w("downsample.conv.weight", True) is not None:
            x = self._conv(x, "downsample", stride=2, pad_mode="replicate")
        return x

    def encode(self, wave: torch.Tensor, quantizers: Optional[int] = None) -> torch.Tensor:
        """-> codes [B, n, frames]."""
        return self.quantize(self.encode_latents(wave), quantizers)

    @torch.no_grad()
    def decode(self, codes: torch.Tensor) -> torch.Tensor:
        """codes [B, n, frames] -> wave [B, 1, frames * samples_per_frame]."""
        cfg = self.cfg
        if codes.dim() == 2:
            codes = codes[None]
        x = self.dequantize(codes)
        if self._w("upsample.conv.weight", True) is not None:
            x = self._conv_t(x, "upsample", 2, groups=cfg.upsample_groups)
        x = self._transformer(x.transpose(1, 2), "decoder_transformer").transpose(1, 2)
        x = self._conv(x, "decoder.layers.0")
        idx = 1
        for ratio in cfg.ratios:
            x = self._conv_t(F.elu(x), f"decoder.layers.{idx + 1}", ratio)
            idx += 2
            for j in range(cfg.residual_layers):
                x = self._resblock(x, f"decoder.layers.{idx}", cfg.dilation_growth ** j)
                idx += 1
        return self._conv(F.elu(x), f"decoder.layers.{idx + 1}")
