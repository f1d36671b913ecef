"""EnCodec decoder: residual-vector-quantised codes -> waveform (the audio end of MusicGen- and
Bark-class models).

codes -> sum of codebook vectors -> conv(k7) -> LSTM (+ skip) -> per ratio [ELU -> transposed conv
(kernel 2 * ratio, trimmed to ratio * length) -> residual blocks (ELU, conv k3 dilated, ELU, conv k1;
conv or identity shortcut)] -> ELU -> conv(k7). Convolutions pad by reflection, on the left only
in the causal models; weight-normalised storage is folded at load.
Reference: src/HartsyInference.Audio/ (codecs).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.nn.functional as F


@dataclass(frozen=True)
class EncodecConfig:
    hidden: int = 128
    filters: int = 32
    ratios: tuple = (8, 5, 4, 2)
    residual_layers: int = 1
    dilation_growth: int = 2
    kernel: int = 7
    last_kernel: int = 7
    residual_kernel: int = 3
    lstm_layers: int = 2
    causal: bool = True
    conv_shortcut: bool = True
    trim_right_ratio: float = 1.0
    pad_mode: str = "reflect"
    sampling_rate: int = 24000

    @staticmethod
    def from_hf(d: dict) -> "EncodecConfig":
        if d.get("norm_type", "weight_norm") != "weight_norm":
            raise ValueError("only weight-normalised EnCodec checkpoints are supported")
        return EncodecConfig(hidden=d.get("hidden_size", 128), filters=d.get("num_filters", 32),
                             ratios=tuple(d.get("upsampling_ratios") or (8, 5, 4, 2)), residual_layers=d.get("num_residual_layers", 1),
                             dilation_growth=d.get("dilation_growth_rate", 2), kernel=d.get("kernel_size", 7),
                             last_kernel=d.get("last_kernel_size", 7), residual_kernel=d.get("residual_kernel_size", 3),
                             lstm_layers=d.get("num_lstm_layers", 2), causal=bool(d.get("use_causal_conv", True)),
                             conv_shortcut=bool(d.get("use_conv_shortcut", True)), trim_right_ratio=float(d.get("trim_right_ratio", 1.0)),
                             pad_mode=d.get("pad_mode", "reflect"), sampling_rate=d.get("sampling_rate", 24000))


class EncodecDecoder:
    def __init__(self, cfg: EncodecConfig, get: Callable[[str], Optional[torch.Tensor]], device="cpu"):
        self.cfg, self.device = cfg, torch.device(device)
        self._get, self._cache = get, {}
        self.lstm = torch.nn.LSTM(cfg.hidden, cfg.hidden, cfg.lstm_layers).to(self.device)
        with torch.no_grad():
            for name, p in self.lstm.named_parameters():
                p.copy_(self._w(f"decoder.layers.1.lstm.{name}"))
        self.lstm.eval()

    def _w(self, name: str) -> torch.Tensor:
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

    def _pad(self, x: torch.Tensor, left: int, right: int) -> torch.Tensor:
        if self.cfg.pad_mode != "reflect":
            return F.pad(x, (left, right), self.cfg.pad_mode)
        extra = max(0, max(left, right) - x.shape[-1] + 1)          # reflection needs more samples than the pad width
        y = F.pad(F.pad(x, (0, extra)), (left, right), "reflect")
        return y[..., : y.shape[-1] - extra]

    def _conv(self, x: torch.Tensor, p: str, dilation: int = 1) -> torch.Tensor:
        w = self._w(p + ".conv.weight")
        total = (w.shape[-1] - 1) * dilation
        left, right = (total, 0) if self.cfg.causal else (total - total // 2, total // 2)
        return F.conv1d(self._pad(x, left, right), w, self._w(p + ".conv.bias"), dilation=dilation)

    def _conv_t(self, x: torch.Tensor, p: str, stride: int) -> torch.Tensor:
        w = self._w(p + ".conv.weight")
        y = F.conv_transpose1d(x, w, self._w(p + ".conv.bias"), stride=stride)
        total = w.shape[-1] - stride
        right = math.ceil(total * self.cfg.trim_right_ratio) if self.cfg.causal else total // 2
        return y[..., total - right: y.shape[-1] - right]

    @torch.no_grad()
    def latents_from_codes(self, codes: torch.Tensor) -> torch.Tensor:
        """codes [B, n, frames] -> [B, hidden, frames]."""
        total = None
        for i in range(codes.shape[1]):
            q = self._w(f"quantizer.layers.{i}.codebook.embed")[codes[:, i].to(self.device)]
            total = q if total is None else total + q
        return total.transpose(1, 2)

    @torch.no_grad()
    def decode_latents(self, z: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        x = self._conv(z.to(self.device).float(), "decoder.layers.0")
        x = (self.lstm(x.permute(2, 0, 1))[0] + x.permute(2, 0, 1)).permute(1, 2, 0)
        idx = 2
        for ratio in cfg.ratios:
            x = self._conv_t(F.elu(x), f"decoder.layers.{idx + 1}", ratio)
            for j in range(cfg.residual_layers):
                p = f"decoder.layers.{idx + 2 + j}"
                y = self._conv(F.elu(x), p + ".block.1", dilation=cfg.dilation_growth ** j)
                y = self._conv(F.elu(y), p + ".block.3")
                x = (self._conv(x, p + ".shortcut") if cfg.conv_shortcut else x) + y
            idx += 2 + cfg.residual_layers
        return self._conv(F.elu(x), f"decoder.layers.{idx + 1}")

    def decode(self, codes: torch.Tensor) -> torch.Tensor:
        """codes [B, n, frames] -> wave [B, channels, frames * prod(ratios)]."""
        if codes.dim() == 2:
            codes = codes[None]
        return self.decode_latents(self.latents_from_codes(codes))
