"""Real-ESRGAN super-resolution: RRDBNet (residual-in-residual dense blocks) and overlapping-tile
inference with linear-ramp blending, so images of any size upscale in bounded memory.

Network: conv_first -> N RRDBs (three dense blocks of five 3x3 convolutions with growing input,
each scaled by 0.2 and added back) -> conv_body (+ skip) -> nearest 2x + conv (twice) -> conv_hr ->
conv_last. The x2 model folds 2x2 pixel blocks into channels first and then runs the x4 body.
Convolutions go through PyTorch (cuDNN); this is off the named hot paths.

Reference: src/HartsyInference.Vision/Upscale/RrdbNet.cs, UpscalePipeline.cs, RealEsrganConverter.cs;
src/HartsyInference.Engine/Services/RestoreService.cs. Tensor names follow the Real-ESRGAN releases
(``conv_first``, ``body.N.rdbM.convK``, ``conv_body``, ``conv_up1/2``, ``conv_hr``, ``conv_last``,
optionally under ``params_ema.``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.nn.functional as F


@dataclass(frozen=True)
class RrdbConfig:
    num_feat: int = 64
    num_block: int = 23
    num_grow: int = 32
    scale: int = 4


X4PLUS = RrdbConfig()
X4PLUS_ANIME_6B = RrdbConfig(num_block=6)
X2PLUS = RrdbConfig(scale=2)


def detect_rrdb_config(keys) -> RrdbConfig:
    """Block count from the tensor names; scale 2 when conv_first takes the 12 folded channels."""
    ks = [k.split("params_ema.")[-1].split("params.")[-1] for k in keys]
    blocks = 1 + max((int(k.split(".")[1]) for k in ks if k.startswith("body.")), default=-1)
    return RrdbConfig(num_block=blocks)


class RrdbNet:
    def __init__(self, cfg: RrdbConfig = X4PLUS, device="cpu", dtype=torch.float32,
                 get: Optional[Callable[[str], Optional[torch.Tensor]]] = None, seed: int = 0):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        g = torch.Generator().manual_seed(seed)
        self.w: dict[str, torch.Tensor] = {}

        def conv(name, co, ci):
            w = b = None
            if get is not None:
                for pre in ("", "params_ema.", "params."):
                    w = get(pre + name + ".weight")
                    if w is not None:
                        b = get(pre + name + ".bias")
                        break
                if w is None:
                    raise KeyError(name + ".weight")
            else:
                w = torch.randn(co, ci, 3, 3, generator=g) * (0.1 / (ci * 9) ** 0.5)
                b = torch.zeros(co)
            self.w[name + ".weight"] = w.to(dtype).to(self.device)
            self.w[name + ".bias"] = b.to(dtype).to(self.device)

        nf, gc = cfg.num_feat, cfg.num_grow
        in_ch = 3 * (4 if cfg.scale == 2 else 16 if cfg.scale == 1 else 1)
        if get is not None:       # the release tells which variant it is
            for pre in ("", "params_ema.", "params."):
                t = get(pre + "conv_first.weight")
                if t is not None:
                    in_ch = t.shape[1]
                    break
        self.unshuffle = {3: 1, 12: 2, 48: 4}[in_ch]
        conv("conv_first", nf, in_ch)
        for i in range(cfg.num_block):
            for r in (1, 2, 3):
                for c in range(1, 6):
                    conv(f"body.{i}.rdb{r}.conv{c}", gc if c < 5 else nf, nf + (c - 1) * gc)
        for n in ("conv_body", "conv_up1", "conv_up2", "conv_hr"):
            conv(n, nf, nf)
        conv("conv_last", 3, nf)

    @property
    def scale(self) -> int:
        return 4 // self.unshuffle

    def _c(self, x, name):
        return F.conv2d(x, self.w[name + ".weight"], self.w[name + ".bias"], padding=1)

    def _rdb(self, x, p):
        feats = [x]
        for c in range(1, 5):
            feats.append(F.leaky_relu(self._c(torch.cat(feats, 1), f"{p}.conv{c}"), 0.2))
        return self._c(torch.cat(feats, 1), f"{p}.conv5") * 0.2 + x

    @torch.no_grad()
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """x [B, 3, H, W] in [0, 1] -> [B, 3, scale H, scale W]."""
        x = x.to(self.device).to(self.dtype)
        if self.unshuffle > 1:
            x = F.pixel_unshuffle(x, self.unshuffle)
        feat = self._c(x, "conv_first")
        body = feat
        for i in range(self.cfg.num_block):
            y = body
            for r in (1, 2, 3):
                y = self._rdb(y, f"body.{i}.rdb{r}")
            body = y * 0.2 + body
        feat = feat + self._c(body, "conv_body")
        feat = F.leaky_relu(self._c(F.interpolate(feat, scale_factor=2, mode="nearest"), "conv_up1"), 0.2)
        feat = F.leaky_relu(self._c(F.interpolate(feat, scale_factor=2, mode="nearest"), "conv_up2"), 0.2)
        return self._c(F.leaky_relu(self._c(feat, "conv_hr"), 0.2), "conv_last").float()


class UpscalePipeline:
    """Whole-image or overlapping-tile upscaling of RGB24 images."""

    def __init__(self, net: RrdbNet, tile: int = 128, overlap: float = 0.25):
        self.net, self.tile, self.overlap = net, tile, overlap

    @torch.no_grad()
    def upscale_tensor(self, img: torch.Tensor) -> torch.Tensor:
        """img [3, H, W] in [0, 1] -> [3, s H, s W] in [0, 1]."""
        s, t = self.net.scale, self.tile
        _, h, w = img.shape
        m = self.net.unshuffle
        if m > 1 and (h % m or w % m):       # folded variants need sizes divisible by the fold
            img = F.pad(img[None], (0, (-w) % m, 0, (-h) % m), mode="replicate")[0]
        hp, wp = img.shape[1:]
        if t <= 0 or (hp <= t and wp <= t):
            return self.net.forward(img[None])[0, :, : h * s, : w * s].clamp(0, 1).cpu()
        step = max(m, int(t * (1 - self.overlap)) // m * m)
        out = torch.zeros(3, hp * s, wp * s)
        weight = torch.zeros(1, hp * s, wp * s)
        ys = list(range(0, max(hp - t, 0) + 1, step))
        xs = list(range(0, max(wp - t, 0) + 1, step))
        if ys[-1] + t < hp:
            ys.append(hp - t)
        if xs[-1] + t < wp:
            xs.append(wp - t)
        for y0 in ys:
            for x0 in xs:
                y1, x1 = min(y0 + t, hp), min(x0 + t, wp)
                up = self.net.forward(img[None, :, y0:y1, x0:x1])[0].cpu()
                th, tw = up.shape[1:]
                # linear ramps over the overlap on the sides that have a neighbour
                ramp = max(int(t * self.overlap) * s, 1)
                wy, wx = torch.ones(th), torch.ones(tw)
                r = torch.linspace(1.0 / (ramp + 1), ramp / (ramp + 1.0), ramp)
                if y0 > 0:
                    wy[:ramp] = r[: min(ramp, th)]
                if y1 < hp:
                    wy[-ramp:] = r.flip(0)[-min(ramp, th):]
                if x0 > 0:
                    wx[:ramp] = r[: min(ramp, tw)]
                if x1 < wp:
                    wx[-ramp:] = r.flip(0)[-min(ramp, tw):]
                wt = (wy[:, None] * wx[None, :])[None]
                out[:, y0 * s:y0 * s + th, x0 * s:x0 * s + tw] += up * wt
                weight[:, y0 * s:y0 * s + th, x0 * s:x0 * s + tw] += wt
        return (out / weight.clamp_min(1e-8))[:, : h * s, : w * s].clamp(0, 1)

    def upscale_rgb(self, rgb: bytes, width: int, height: int) -> tuple[bytes, int, int]:
        img = torch.frombuffer(bytearray(rgb), dtype=torch.uint8).reshape(height, width, 3).permute(2, 0, 1).float() / 255.0
        up = self.upscale_tensor(img)
        u8 = (up * 255.0).round().to(torch.uint8).permute(1, 2, 0).contiguous()
        return u8.numpy().tobytes(), up.shape[2], up.shape[1]
