"""Depth Anything: a DINOv2 backbone tapped at four depths, a DPT neck (reassemble each tap into an
image-like map at its own scale, fuse them coarse to fine with pre-activation residual units and
bilinear upsampling) and a three-convolution head that predicts relative (ReLU) or metric
(sigmoid x max depth) depth at the input resolution.

The backbone runs on the framework's transformer ops; the neck and head are small convolutions
through PyTorch.

Reference: src/HartsyInference.Vision/DepthAnything/. Tensor names follow Hugging Face
``DepthAnythingForDepthEstimation`` (``backbone.*``, ``neck.*``, ``head.*``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.nn.functional as F

from ..encoders.vit import VitConfig, VitEncoder, vit_from_hf


@dataclass(frozen=True)
class DepthAnythingConfig:
    backbone: VitConfig
    taps: tuple = (3, 6, 9, 12)                  # 1-based block counts whose states feed the neck
    reassemble_hidden: int = 384
    neck_sizes: tuple = (48, 96, 192, 384)
    factors: tuple = (4, 2, 1, 0.5)
    fusion: int = 64
    head_hidden: int = 32
    metric: bool = False
    max_depth: float = 1.0


def depth_anything_from_hf(d: dict) -> DepthAnythingConfig:
    bc = dict(d["backbone_config"])
    bc["model_type"] = "dinov2"
    layers = bc["num_hidden_layers"]
    taps = bc.get("out_indices") or [layers]
    if bc.get("out_features") and not bc.get("out_indices"):
        taps = [int(str(f).replace("stage", "")) for f in bc["out_features"]]
    return DepthAnythingConfig(backbone=vit_from_hf(bc), taps=tuple(int(t) for t in taps),
                               reassemble_hidden=d.get("reassemble_hidden_size", 384), neck_sizes=tuple(d.get("neck_hidden_sizes", (48, 96, 192, 384))),
                               factors=tuple(d.get("reassemble_factors", (4, 2, 1, 0.5))), fusion=d.get("fusion_hidden_size", 64),
                               head_hidden=d.get("head_hidden_size", 32), metric=d.get("depth_estimation_type", "relative") == "metric",
                               max_depth=float(d.get("max_depth") or 1.0))


class DepthAnything:
    def __init__(self, cfg: DepthAnythingConfig, device="cpu", get: Optional[Callable[[str], Optional[torch.Tensor]]] = None, seed: int = 0):
        self.cfg, self.device = cfg, torch.device(device)
        bget = None
        if get is not None:
            def bget(name):          # the backbone's tensors sit under "backbone."
                return get("backbone." + name)
        self.backbone = VitEncoder(cfg.backbone, device, get=bget, seed=seed, prefix="")
        self._get = get
        self._g = torch.Generator().manual_seed(seed + 7)
        self.w: dict[str, torch.Tensor] = {}

    def _p(self, name: str, *shape) -> Optional[torch.Tensor]:
        if name in self.w:
            return self.w[name]
        t = self._get(name) if self._get is not None else None
        if t is None:
            if self._get is not None:
                if name.endswith(".bias"):
                    self.w[name] = None
                    return None
                raise KeyError(name)
            fan = 1
            for s in shape[1:]:
                fan *= s
            t = torch.zeros(*shape) if name.endswith(".bias") else torch.randn(*shape, generator=self._g) * (1.0 / max(fan, 1)) ** 0.5
        self.w[name] = t.float().to(self.device)
        return self.w[name]

    def _conv(self, x, name, co, ci, k, stride=1, padding=0):
        return F.conv2d(x, self._p(name + ".weight", co, ci, k, k), self._p(name + ".bias", co), stride=stride, padding=padding)

    def _residual(self, x, p, c):
        y = self._conv(torch.relu(x), p + ".convolution1", c, c, 3, padding=1)
        y = self._conv(torch.relu(y), p + ".convolution2", c, c, 3, padding=1)
        return x + y

    @torch.no_grad()
    def predict(self, image: torch.Tensor) -> torch.Tensor:
        """image [3, H, W] normalised (ImageNet statistics), H and W multiples of the patch size ->
        depth [H, W] (fp32)."""
        cfg = self.cfg
        P = cfg.backbone.patch
        gh, gw = image.shape[-2] // P, image.shape[-1] // P
        states = self.backbone.hidden_states(image, taps=list(cfg.taps))
        feats = []
        for i, (st, ch, fac) in enumerate(zip(states, cfg.neck_sizes, cfg.factors)):
            x = st[1:].float().reshape(1, gh, gw, -1).permute(0, 3, 1, 2)
            p = f"neck.reassemble_stage.layers.{i}."
            x = self._conv(x, p + "projection", ch, cfg.reassemble_hidden, 1)
            if fac > 1:
                k = int(fac)
                x = F.conv_transpose2d(x, self._p(p + "resize.weight", ch, ch, k, k), self._p(p + "resize.bias", ch), stride=k)
            elif fac < 1:
                x = self._conv(x, p + "resize", ch, ch, 3, stride=int(1 / fac), padding=1)
            feats.append(F.conv2d(x, self._p(f"neck.convs.{i}.weight", cfg.fusion, ch, 3, 3), None, padding=1))
        feats = feats[::-1]                                  # coarsest first
        fused = None
        c = cfg.fusion
        for i, f in enumerate(feats):
            p = f"neck.fusion_stage.layers.{i}."
            size = feats[i + 1].shape[2:] if i + 1 < len(feats) else None
            if fused is None:
                h = f
            else:
                if fused.shape != f.shape:
                    f = F.interpolate(f, size=fused.shape[2:], mode="bilinear", align_corners=False)
                h = fused + self._residual(f, p + "residual_layer1", c)
            h = self._residual(h, p + "residual_layer2", c)
            h = F.interpolate(h, size=tuple(size), mode="bilinear", align_corners=True) if size is not None else \
                F.interpolate(h, scale_factor=2, mode="bilinear", align_corners=True)
            fused = self._conv(h, p + "projection", c, c, 1)
        d = self._conv(fused, "head.conv1", c // 2, c, 3, padding=1)
        d = F.interpolate(d, size=(gh * P, gw * P), mode="bilinear", align_corners=True)
        d = torch.relu(self._conv(d, "head.conv2", cfg.head_hidden, c // 2, 3, padding=1))
        d = self._conv(d, "head.conv3", 1, cfg.head_hidden, 1)
        d = torch.sigmoid(d) * cfg.max_depth if cfg.metric else torch.relu(d)
        return d[0, 0]
