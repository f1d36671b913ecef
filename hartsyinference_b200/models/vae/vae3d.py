"""Causal 3-D VAE decoder (Wan 2.1 layout): causal 3x3x3 convolutions (temporal padding on the past
side only), channel-RMS-norm residual blocks, a spatial attention mid block, and up-sampling
stages that double space (nearest + conv) and, for the first two, time (a temporal convolution to
2C channels interleaved into frames). 4x temporal and 8x spatial expansion: latent [16, T, h, w] ->
video [3, 4(T - 1) + 1, 8h, 8w].

Reference: src/HartsyInference.Diffusion/Models/Vae/CausalConv3d.cs (fast path :146-174 = padded
frames + kt 2-D convolutions + tap accumulation) and the Wan VAE decoder files beside it. The
convolutions run as one shifted-row tcgen05 GEMM per layer on CUDA (``ops.causal_conv3d``) and
through PyTorch's conv3d on CPU."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.nn.functional as F


@dataclass(frozen=True)
class Vae3dConfig:
    z_dim: int = 16
    dim: int = 96
    dim_mult: tuple = (1, 2, 4, 4)
    num_res_blocks: int = 2
    temporal_upsample: tuple = (True, True, False)
    out_channels: int = 3


WAN_VAE = Vae3dConfig()


def tiny_vae3d() -> Vae3dConfig:
    return Vae3dConfig(z_dim=4, dim=8, dim_mult=(1, 2, 2), num_res_blocks=1, temporal_upsample=(True, False))


class Vae3dDecoder:
    def __init__(self, cfg: Vae3dConfig = WAN_VAE, device="cpu", dtype=torch.bfloat16,
                 get: Optional[Callable[[str], Optional[torch.Tensor]]] = None, seed: int = 0):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        self._get, self._g = get, torch.Generator().manual_seed(seed)
        self.w: dict[str, torch.Tensor] = {}
        self._packed: dict[str, torch.Tensor] = {}      # conv weights in the GEMM layout, built on first use
        dims = [cfg.dim * m for m in [cfg.dim_mult[-1]] + list(reversed(cfg.dim_mult))]
        self._conv3("conv2", cfg.z_dim, cfg.z_dim, 1)
        self._conv3("decoder.conv1", dims[0], cfg.z_dim, 3)
        self._res("decoder.middle.0", dims[0], dims[0])
        self._attn("decoder.middle.1", dims[0])
        self._res("decoder.middle.2", dims[0], dims[0])
        self.stages = []
        idx = 0
        for i, (ci, co) in enumerate(zip(dims[:-1], dims[1:])):
            if i in (1, 2, 3):
                ci = ci // 2
            blocks = []
            for _ in range(cfg.num_res_blocks + 1):
                name = f"decoder.upsamples.{idx}"
                self._res(name, ci, co)
                blocks.append((name, ci, co))
                ci = co
                idx += 1
            up = None
            if i != len(cfg.dim_mult) - 1:
                name = f"decoder.upsamples.{idx}"
                temporal = cfg.temporal_upsample[i]
                self._p(name + ".resample.1.weight", (co // 2, co, 3, 3))
                self._p(name + ".resample.1.bias", (co // 2,), zeros=True)
                if temporal:
                    self._conv3(name + ".time_conv", co * 2, co, (3, 1, 1))
                up = (name, temporal)
                idx += 1
            self.stages.append((blocks, up))
        self._p("decoder.head.0.gamma", (dims[-1],), ones=True)
        self._conv3("decoder.head.2", cfg.out_channels, dims[-1], 3)

    def _p(self, name, shape, ones=False, zeros=False):
        t = self._get(name) if self._get is not None else None
        if t is None:
            if ones:
                t = torch.ones(shape)
            elif zeros:
                t = torch.zeros(shape)
            else:
                fan = 1
                for s in shape[1:]:
                    fan *= s
                t = torch.randn(shape, generator=self._g) * (1.0 / max(fan, 1)) ** 0.5
        self.w[name] = t.reshape(shape).to(self.dtype).to(self.device)

    def _conv3(self, name, co, ci, k):
        k = (k, k, k) if isinstance(k, int) else k
        self._p(name + ".weight", (co, ci) + tuple(k))
        self._p(name + ".bias", (co,), zeros=True)

    def _res(self, name, ci, co):
        self._p(name + ".residual.0.gamma", (ci,), ones=True)
        self._conv3(name + ".residual.2", co, ci, 3)
        self._p(name + ".residual.3.gamma", (co,), ones=True)
        self._conv3(name + ".residual.6", co, co, 3)
        if ci != co:
            self._conv3(name + ".shortcut", co, ci, 1)

    def _attn(self, name, c):
        self._p(name + ".norm.gamma", (c,), ones=True)
        self._p(name + ".to_qkv.weight", (3 * c, c, 1, 1))
        self._p(name + ".to_qkv.bias", (3 * c,), zeros=True)
        self._p(name + ".proj.weight", (c, c, 1, 1))
        self._p(name + ".proj.bias", (c,), zeros=True)

    # -- ops ----------------------------------------------------------------------------
    def causal_conv3d(self, x, name):
        """x [B, C, T, H, W]; pads (kt - 1) frames on the past side, (k - 1) / 2 spatially."""
        w, b = self.w[name + ".weight"], self.w[name + ".bias"]
        kt, kh, kw = w.shape[2:]
        if x.is_cuda and x.shape[0] == 1 and x.dtype == torch.bfloat16 and w.shape[1] >= 16:
            # one tcgen05 GEMM over the padded channels-last volume (weights packed once)
            from ... import ops
            packed = self._packed.get(name)
            if packed is None:
                packed = self._packed[name] = ops.core.pack_conv3d_weight(w)
            return ops.causal_conv3d(x, w, b, packed=packed)
        x = F.pad(x, (kw // 2, kw // 2, kh // 2, kh // 2, kt - 1, 0))
        return F.conv3d(x, w, b)

    def rms_norm(self, x, name):
        """Channel-wise L2 normalisation times sqrt(C) times gamma (Wan ``RMS_norm``)."""
        g = self.w[name + ".gamma"]
        shape = (1, -1) + (1,) * (x.dim() - 2)
        return (F.normalize(x.float(), dim=1) * (x.shape[1] ** 0.5)).to(x.dtype) * g.reshape(shape)

    def _resblock(self, x, name, ci, co):
        h = self.causal_conv3d(F.silu(self.rms_norm(x, name + ".residual.0")), name + ".residual.2")
        h = self.causal_conv3d(F.silu(self.rms_norm(h, name + ".residual.3")), name + ".residual.6")
        if ci != co:
            x = self.causal_conv3d(x, name + ".shortcut")
        return x + h

    def _attention(self, x, name):
        b, c, t, hh, ww = x.shape
        y = x.permute(0, 2, 1, 3, 4).reshape(b * t, c, hh, ww)
        y = self.rms_norm(y, name + ".norm")
        qkv = F.conv2d(y, self.w[name + ".to_qkv.weight"], self.w[name + ".to_qkv.bias"])
        q, k, v = qkv.reshape(b * t, 1, 3 * c, hh * ww).permute(0, 1, 3, 2).chunk(3, dim=-1)
        o = F.scaled_dot_product_attention(q, k, v)
        o = o.squeeze(1).permute(0, 2, 1).reshape(b * t, c, hh, ww)
        o = F.conv2d(o, self.w[name + ".proj.weight"], self.w[name + ".proj.bias"])
        return x + o.reshape(b, t, c, hh, ww).permute(0, 2, 1, 3, 4)

    def _upsample(self, x, name, temporal):
        b, c, t, hh, ww = x.shape
        if temporal and t > 1:
            # the first frame is kept single, every later frame becomes two
            first, rest = x[:, :, :1], x
            y = self.causal_conv3d(rest, name + ".time_conv")              # [B, 2C, T, H, W]
            y = y.reshape(b, 2, c, t, hh, ww)
            y = torch.stack([y[:, 0], y[:, 1]], dim=3).reshape(b, c, 2 * t, hh, ww)
            x = y[:, :, 1:]                                                # 2T - 1 frames
            t = x.shape[2]
        y = x.permute(0, 2, 1, 3, 4).reshape(b * t, c, hh, ww)
        y = F.interpolate(y.float(), scale_factor=2.0, mode="nearest").to(x.dtype)
        y = F.conv2d(y, self.w[name + ".resample.1.weight"], self.w[name + ".resample.1.bias"], padding=1)
        return y.reshape(b, t, c // 2, 2 * hh, 2 * ww).permute(0, 2, 1, 3, 4)

    @torch.no_grad()
    def decode(self, z: torch.Tensor) -> torch.Tensor:
        """z [B, z_dim, T, h, w] -> video [B, 3, T', 8h, 8w] in [-1, 1] (float32)."""
        x = self.causal_conv3d(z.to(self.device).to(self.dtype), "conv2")
        x = self.causal_conv3d(x, "decoder.conv1")
        c0 = x.shape[1]
        x = self._resblock(x, "decoder.middle.0", c0, c0)
        x = self._attention(x, "decoder.middle.1")
        x = self._resblock(x, "decoder.middle.2", c0, c0)
        for blocks, up in self.stages:
            for name, ci, co in blocks:
                x = self._resblock(x, name, ci, co)
            if up is not None:
                x = self._upsample(x, up[0], up[1])
        x = self.causal_conv3d(F.silu(self.rms_norm(x, "decoder.head.0")), "decoder.head.2")
        return x.float().clamp(-1, 1)
