"""Descript Audio Codec (DAC): waveform <-> residual-vector-quantised codes.

Encoder: conv(k7) -> per stage [3 residual units (snake, dilated conv k7 with dilation 1 / 3 / 9,
snake, conv k1) -> snake -> strided conv (kernel 2 * stride)] -> snake -> conv(k3).
Quantiser: ``n_codebooks`` stages on the running residual; each projects to a small code space,
picks the nearest code by cosine similarity and projects the code back.
Decoder: conv(k7) -> per stage [snake -> transposed conv -> 3 residual units] -> snake -> conv(k7) -> tanh.
snake(x) = x + sin^2(alpha x) / alpha with one alpha per channel.

Convolutions stored with weight normalisation are folded at load. The codec is the token <-> audio
end of the codec language-model speech and music families.
Reference: src/HartsyInference.Audio/ (codecs).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.nn.functional as F


@dataclass(frozen=True)
class DacConfig:
    encoder_hidden: int = 64
    decoder_hidden: int = 1536
    hidden: int = 1024
    down: tuple = (2, 4, 8, 8)
    up: tuple = (8, 8, 4, 2)
    n_codebooks: int = 9
    codebook_size: int = 1024
    codebook_dim: int = 8
    sampling_rate: int = 44100

    @property
    def hop(self) -> int:
        return math.prod(self.down)

    @staticmethod
    def from_hf(d: dict) -> "DacConfig":
        down = tuple(d.get("downsampling_ratios") or (2, 4, 8, 8))
        enc = d.get("encoder_hidden_size", 64)
        return DacConfig(encoder_hidden=enc, decoder_hidden=d.get("decoder_hidden_size", 1536),
                         hidden=d.get("hidden_size") or enc * 2 ** len(down), down=down,
                         up=tuple(d.get("upsampling_ratios") or down[::-1]), n_codebooks=d.get("n_codebooks", 9),
                         codebook_size=d.get("codebook_size", 1024), codebook_dim=d.get("codebook_dim", 8),
                         sampling_rate=d.get("sampling_rate", 44100))


def snake(x: torch.Tensor, alpha: torch.Tensor) -> torch.Tensor:
    return x + torch.sin(alpha * x).pow(2) / (alpha + 1e-9)


class DacCodec:
    def __init__(self, cfg: DacConfig, get: Callable[[str], Optional[torch.Tensor]], device="cpu", final_tanh: bool = True,
                 odd_stride_padding: bool = False):
        """``final_tanh`` False and ``odd_stride_padding`` True give the decoder variant X-Codec uses (no output
        squashing; transposed convolutions of odd stride emit one more sample so that lengths stay multiples of the hop)."""
        self.cfg, self.device = cfg, torch.device(device)
        self._get, self._cache = get, {}
        self.final_tanh, self.odd_stride_padding = final_tanh, odd_stride_padding

    def _w(self, name: str) -> torch.Tensor:
        """fp32 tensor ``name``; a weight-normalised convolution (g * v / |v| per output channel) is folded."""
        hit = self._cache.get(name)
        if hit is not None:
            return hit
        t = self._get(name)
        if t is None and name.endswith(".weight"):
            stem = name[: -len(".weight")]
            g, v = self._get(stem + ".parametrizations.weight.original0"), self._get(stem + ".parametrizations.weight.original1")
            if g is None:
                g, v = self._get(stem + ".weight_g"), self._get(stem + ".weight_v")
            if g is not None and v is not None:
                v = v.float()
                t = v * (g.float() / v.flatten(1).norm(dim=1).reshape(-1, *([1] * (v.dim() - 1))))
        if t is None:
            raise KeyError(f"missing tensor {name}")
        t = t.float().to(self.device)
        self._cache[name] = t
        return t

    def _conv(self, x, p, **kw):
        return F.conv1d(x, self._w(p + ".weight"), self._w(p + ".bias"), **kw)

    def _res(self, x: torch.Tensor, p: str, dilation: int) -> torch.Tensor:
        y = self._conv(snake(x, self._w(p + ".snake1.alpha")), p + ".conv1", dilation=dilation, padding=3 * dilation)
        y = self._conv(snake(y, self._w(p + ".snake2.alpha")), p + ".conv2")
        return x + y

    # ------------------------------------------------------------------------------------ parts
    @torch.no_grad()
    def encode_latents(self, wave: torch.Tensor, pad_to_hop: bool = True) -> torch.Tensor:
        """wave [B, samples] -> continuous latents [B, hidden, frames] (the input is zero-padded to a whole hop)."""
        x = wave.to(self.device).float()
        x = (F.pad(x, (0, (-x.shape[-1]) % self.cfg.hop)) if pad_to_hop else x)[:, None]
        x = self._conv(x, "encoder.conv1", padding=3)
        for i, s in enumerate(self.cfg.down):
            p = f"encoder.block.{i}"
            for j, dil in enumerate((1, 3, 9)):
                x = self._res(x, f"{p}.res_unit{j + 1}", dil)
            x = self._conv(snake(x, self._w(p + ".snake1.alpha")), p + ".conv1", stride=s, padding=math.ceil(s / 2))
        return self._conv(snake(x, self._w("encoder.snake1.alpha")), "encoder.conv2", padding=1)

    @torch.no_grad()
    def quantize(self, latents: torch.Tensor, n_codebooks: Optional[int] = None) -> tuple[torch.Tensor, torch.Tensor]:
        """latents [B, hidden, frames] -> (codes [B, n, frames] int64, quantised latents)."""
        n = n_codebooks or self.cfg.n_codebooks
        residual, total, codes = latents, torch.zeros_like(latents), []
        for i in range(n):
            p = f"quantizer.quantizers.{i}"
            z = self._conv(residual, p + ".in_proj")                                     # [B, cd, T]
            b, cd, t = z.shape
            book = self._w(p + ".codebook.weight")
            sim = F.normalize(z.permute(0, 2, 1).reshape(b * t, cd)) @ F.normalize(book).t()
            idx = sim.argmax(1).reshape(b, t)
            q = self._conv(book[idx].transpose(1, 2), p + ".out_proj")
            total, residual = total + q, residual - q
            codes.append(idx)
        return torch.stack(codes, 1), total

    @torch.no_grad()
    def latents_from_codes(self, codes: torch.Tensor) -> torch.Tensor:
        total = None
        for i in range(codes.shape[1]):
            p = f"quantizer.quantizers.{i}"
            q = self._conv(self._w(p + ".codebook.weight")[codes[:, i].to(self.device)].transpose(1, 2), p + ".out_proj")
            total = q if total is None else total + q
        return total

    @torch.no_grad()
    def decode_latents(self, z: torch.Tensor) -> torch.Tensor:
        """quantised latents [B, hidden, frames] -> wave [B, frames * hop] in [-1, 1]."""
        x = self._conv(z.to(self.device).float(), "decoder.conv1", padding=3)
        for i, s in enumerate(self.cfg.up):
            p = f"decoder.block.{i}"
            x = F.conv_transpose1d(snake(x, self._w(p + ".snake1.alpha")), self._w(p + ".conv_t1.weight"), self._w(p + ".conv_t1.bias"),
                                   stride=s, padding=math.ceil(s / 2), output_padding=s % 2 if self.odd_stride_padding else 0)
            for j, dil in enumerate((1, 3, 9)):
                x = self._res(x, f"{p}.res_unit{j + 1}", dil)
        x = self._conv(snake(x, self._w("decoder.snake1.alpha")), "decoder.conv2", padding=3)
        return (torch.tanh(x) if self.final_tanh else x)[:, 0]

    # ------------------------------------------------------------------------------------ public
    def encode(self, wave: torch.Tensor, n_codebooks: Optional[int] = None) -> torch.Tensor:
        """wave [B, samples] (or [samples]) -> codes [B, n_codebooks, frames]."""
        if wave.dim() == 1:
            wave = wave[None]
        return self.quantize(self.encode_latents(wave), n_codebooks)[0]

    def decode(self, codes: torch.Tensor) -> torch.Tensor:
        """codes [B, n, frames] -> wave [B, frames * hop]."""
        if codes.dim() == 2:
            codes = codes[None]
        return self.decode_latents(self.latents_from_codes(codes))
