"""UperNet semantic segmentation (scene parsing, the "segmentation map" annotator for control images).

A Swin backbone gives four maps (strides 4 to 32). The head: a pyramid-pooling module on the coarsest
map (average pools to 1, 2, 3 and 6 cells, each through a 1 x 1 convolution, up-sampled and
concatenated with the map, fused by a 3 x 3 convolution), lateral 1 x 1 convolutions on the other
maps, a top-down pass that adds every level to the next finer one, a 3 x 3 convolution per level,
everything up-sampled to the finest level, concatenated, fused, classified per pixel and
up-sampled to the picture. Every convolution is bias-free with BatchNorm (folded at load) and ReLU.
Weights by the `transformers` names (``backbone.*``, ``decode_head.*``). Reference:
src/HartsyInference.Vision/ (annotators: UperNet).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.nn.functional as F

from ..encoders.swin import SwinBackbone, SwinConfig


@dataclass(frozen=True)
class UperNetConfig:
    hidden: int = 512
    labels: int = 150
    pool_scales: tuple = (1, 2, 3, 6)
    swin: SwinConfig = SwinConfig(out_stages=(1, 2, 3, 4))

    @staticmethod
    def from_hf(d: dict) -> "UperNetConfig":
        b = d.get("backbone_config", {})
        if b.get("model_type", "swin") != "swin":
            raise ValueError(f"UperNet backbone '{b.get('model_type')}' is not built (Swin is)")
        labels = d.get("num_labels") or len(d.get("id2label") or {}) or 150
        return UperNetConfig(hidden=d.get("hidden_size", 512), labels=labels, pool_scales=tuple(d.get("pool_scales", (1, 2, 3, 6))),
                             swin=SwinConfig.from_hf(b))


class UperNet:
    def __init__(self, cfg: UperNetConfig, get: Callable[[str], Optional[torch.Tensor]], device="cpu", dtype: torch.dtype = torch.float32):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        self._get, self._folded = get, {}
        self.backbone = SwinBackbone(cfg.swin, get, device, dtype, prefix="backbone.")

    def _conv(self, x, p: str, k: int):
        hit = self._folded.get(p)
        if hit is None:
            g = lambda n: self._get(f"{p}.{n}").float()
            s = g("batch_norm.weight") * torch.rsqrt(g("batch_norm.running_var") + 1e-5)
            hit = ((g("conv.weight") * s[:, None, None, None]).to(self.device).to(self.dtype),
                   (g("batch_norm.bias") - g("batch_norm.running_mean") * s).to(self.device).to(self.dtype))
            self._folded[p] = hit
        return F.relu(F.conv2d(x, hit[0], hit[1], padding=k // 2))

    @torch.no_grad()
    def logits(self, pixels: torch.Tensor) -> torch.Tensor:
        """pixels [B, 3, H, W] (ImageNet-normalised) -> class logits [B, labels, H, W] in fp32."""
        cfg = self.cfg
        maps = self.backbone(pixels)
        up = lambda t, size: F.interpolate(t, size=size, mode="bilinear", align_corners=False)
        top = maps[-1]
        pooled = [top] + [up(self._conv(F.adaptive_avg_pool2d(top, s), f"decode_head.psp_modules.{i}.1", 1), top.shape[-2:])
                          for i, s in enumerate(cfg.pool_scales)]
        laterals = [self._conv(m, f"decode_head.lateral_convs.{i}", 1) for i, m in enumerate(maps[:-1])]
        laterals.append(self._conv(torch.cat(pooled, 1), "decode_head.bottleneck", 3))
        for i in range(len(laterals) - 1, 0, -1):
            laterals[i - 1] = laterals[i - 1] + up(laterals[i], laterals[i - 1].shape[-2:])
        outs = [self._conv(l, f"decode_head.fpn_convs.{i}", 3) for i, l in enumerate(laterals[:-1])] + [laterals[-1]]
        outs = [outs[0]] + [up(o, outs[0].shape[-2:]) for o in outs[1:]]
        y = self._conv(torch.cat(outs, 1), "decode_head.fpn_bottleneck", 3)
        y = F.conv2d(y, self._get("decode_head.classifier.weight").to(self.device).to(self.dtype),
                     self._get("decode_head.classifier.bias").to(self.device).to(self.dtype))
        return up(y.float(), pixels.shape[-2:])

    def segment(self, pixels: torch.Tensor) -> torch.Tensor:
        """-> label map [B, H, W] (int64)."""
        return self.logits(pixels).argmax(1)
