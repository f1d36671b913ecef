"""Vocos: a vocoder that predicts the complex spectrogram and inverts it with one inverse STFT instead
of up-sampling in the time domain (mel or codec features -> 24 kHz audio at one network pass per frame).

backbone: a 7-tap convolution from the input features, LayerNorm, then ConvNeXt blocks (depthwise
7-tap convolution, LayerNorm, 3 x widening Linear, GELU, Linear back, a learned per-channel scale,
residual), a final LayerNorm. head: a Linear to ``n_fft + 2`` values per frame = log-magnitude and
phase of the ``n_fft / 2 + 1`` bins; the magnitude is ``exp`` clipped at 100, the spectrum
``mag (cos p + i sin p)``; the inverse STFT uses a Hann window and centre padding, giving
``(frames - 1) x hop`` samples. Weights by the names of the released checkpoints
(``backbone.embed``, ``backbone.convnext.N.*``, ``head.out``). The released mel model (100 mels,
width 512, 8 blocks, n_fft 1024, hop 256) has 13,531,650 parameters.
Reference: src/HartsyInference.Audio/Models/Vocoders/ (Vocos, VocosConfig, IStft), Codecs/Vocos.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.nn.functional as F


@dataclass(frozen=True)
class VocosConfig:
    in_channels: int = 100
    dim: int = 512
    intermediate: int = 1536
    layers: int = 8
    n_fft: int = 1024
    hop: int = 256
    sampling_rate: int = 24000

    @staticmethod
    def from_dict(d: dict) -> "VocosConfig":
        b = (d.get("backbone") or {}).get("init_args", d)
        h = (d.get("head") or {}).get("init_args", d)
        return VocosConfig(in_channels=b.get("input_channels", 100), dim=b.get("dim", 512), intermediate=b.get("intermediate_dim", 1536),
                           layers=b.get("num_layers", 8), n_fft=h.get("n_fft", 1024), hop=h.get("hop_length", 256),
                           sampling_rate=(d.get("feature_extractor") or {}).get("init_args", d).get("sample_rate", 24000))


class Vocos:
    def __init__(self, cfg: VocosConfig = VocosConfig(), get: Optional[Callable[[str], Optional[torch.Tensor]]] = None, device="cpu",
                 dtype: torch.dtype = torch.float32, seed: int = 0):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        self._get, self._g, self._w = get, torch.Generator().manual_seed(seed), {}

    def _t(self, name: str, shape: tuple, kind: str = "weight") -> torch.Tensor:
        t = self._w.get(name)
        if t is None:
            raw = self._get(name) if self._get is not None else None
            if raw is None:
                if self._get is not None:
                    raise KeyError(name)
                fan = 1
                for s in shape[1:]:
                    fan *= s
                raw = {"ones": torch.ones(shape), "zeros": torch.zeros(shape)}.get(kind)
                if raw is None:
                    raw = torch.randn(shape, generator=self._g) * (1.0 / max(fan, 1)) ** 0.5
            t = raw.reshape(shape).to(self.device).to(self.dtype)
            self._w[name] = t
        return t

    def _ln(self, x, p: str):
        c = self.cfg.dim
        return F.layer_norm(x, (c,), self._t(p + ".weight", (c,), "ones"), self._t(p + ".bias", (c,), "zeros"), 1e-6)

    @torch.no_grad()
    def spectrum(self, features: torch.Tensor) -> torch.Tensor:
        """features [B, in_channels, frames] -> complex spectrum [B, n_fft / 2 + 1, frames]."""
        cfg = self.cfg
        c, m = cfg.dim, cfg.intermediate
        x = F.conv1d(features.to(self.device).to(self.dtype), self._t("backbone.embed.weight", (c, cfg.in_channels, 7)),
                     self._t("backbone.embed.bias", (c,), "zeros"), padding=3)
        x = self._ln(x.transpose(1, 2), "backbone.norm").transpose(1, 2)
        for i in range(cfg.layers):
            p = f"backbone.convnext.{i}"
            y = F.conv1d(x, self._t(p + ".dwconv.weight", (c, 1, 7)), self._t(p + ".dwconv.bias", (c,), "zeros"), padding=3, groups=c)
            y = self._ln(y.transpose(1, 2), p + ".norm")
            y = F.linear(F.gelu(F.linear(y, self._t(p + ".pwconv1.weight", (m, c)), self._t(p + ".pwconv1.bias", (m,), "zeros"))),
                         self._t(p + ".pwconv2.weight", (c, m)), self._t(p + ".pwconv2.bias", (c,), "zeros"))
            x = x + (y * self._t(p + ".gamma", (c,), "ones")).transpose(1, 2)
        x = self._ln(x.transpose(1, 2), "backbone.final_layer_norm")
        out = F.linear(x, self._t("head.out.weight", (cfg.n_fft + 2, c)), self._t("head.out.bias", (cfg.n_fft + 2,), "zeros")).float()
        mag, phase = out.transpose(1, 2).chunk(2, 1)
        mag = torch.exp(mag).clamp(max=1e2)
        return torch.complex(mag * torch.cos(phase), mag * torch.sin(phase))

    @torch.no_grad()
    def __call__(self, features: torch.Tensor) -> torch.Tensor:
        """-> wave [B, (frames - 1) * hop]."""
        cfg = self.cfg
        spec = self.spectrum(features)
        return torch.istft(spec, cfg.n_fft, cfg.hop, cfg.n_fft, torch.hann_window(cfg.n_fft, device=spec.device), center=True)
