"""2-D VAE decoder (AutoencoderKL layout used by Flux and the SD families): conv_in, mid block
(ResNet, single-head attention, ResNet), four up blocks of ResNets with nearest-2x upsampling,
GroupNorm + SiLU, conv_out. Reference: src/HartsyInference.Diffusion/Models/Vae/VaeDecoder.cs (663).
Convolutions and GroupNorm run through PyTorch (cuDNN); they are off the named hot paths."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.nn.functional as F


@dataclass(frozen=True)
class Vae2dConfig:
    latent_channels: int = 16
    block_out_channels: tuple = (128, 256, 512, 512)
    layers_per_block: int = 2
    out_channels: int = 3
    norm_groups: int = 32
    scaling_factor: float = 0.3611
    shift_factor: float = 0.1159


FLUX_VAE = Vae2dConfig()


def tiny_vae2d() -> Vae2dConfig:
    return Vae2dConfig(latent_channels=4, block_out_channels=(8, 16, 16, 16), layers_per_block=1, norm_groups=4)


class Vae2dDecoder:
    def __init__(self, cfg: Vae2dConfig = FLUX_VAE, device="cpu", dtype=torch.bfloat16,
                 get: Optional[Callable[[str], Optional[torch.Tensor]]] = None, seed: int = 0):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        self._get = get
        self._g = torch.Generator().manual_seed(seed)
        self.w: dict[str, torch.Tensor] = {}
        ch = list(cfg.block_out_channels)
        top = ch[-1]
        self._conv("decoder.conv_in", top, cfg.latent_channels, 3)
        self._resnet("decoder.mid_block.resnets.0", top, top)
        self._attn("decoder.mid_block.attentions.0", top)
        self._resnet("decoder.mid_block.resnets.1", top, top)
        prev = top
        self.up: list[tuple[list[tuple[str, int, int]], Optional[str]]] = []
        for i, c in enumerate(reversed(ch)):
            blocks = []
            for j in range(cfg.layers_per_block + 1):
                name = f"decoder.up_blocks.{i}.resnets.{j}"
                self._resnet(name, prev, c)
                blocks.append((name, prev, c))
                prev = c
            up = None
            if i < len(ch) - 1:
                up = f"decoder.up_blocks.{i}.upsamplers.0.conv"
                self._conv(up, c, c, 3)
            self.up.append((blocks, up))
        self._norm("decoder.conv_norm_out", prev)
        self._conv("decoder.conv_out", cfg.out_channels, prev, 3)

    # -- parameters ---------------------------------------------------------------------
    def _p(self, name: str, shape, init: str) -> None:
        t = self._get(name) if self._get is not None else None
        if t is None:
            if init == "ones":
                t = torch.ones(shape)
            elif init == "zeros":
                t = torch.zeros(shape)
            else:
                fan = 1
                for s in shape[1:]:
                    fan *= s
                t = torch.randn(shape, generator=self._g) * (1.0 / max(fan, 1)) ** 0.5
        self.w[name] = t.to(self.dtype).to(self.device)

    def _conv(self, name, co, ci, k):
        self._p(name + ".weight", (co, ci, k, k), "rand")
        self._p(name + ".bias", (co,), "zeros")

    def _norm(self, name, c):
        self._p(name + ".weight", (c,), "ones")
        self._p(name + ".bias", (c,), "zeros")

    def _resnet(self, name, ci, co):
        self._norm(name + ".norm1", ci)
        self._conv(name + ".conv1", co, ci, 3)
        self._norm(name + ".norm2", co)
        self._conv(name + ".conv2", co, co, 3)
        if ci != co:
            self._conv(name + ".conv_shortcut", co, ci, 1)

    def _attn(self, name, c):
        self._norm(name + ".group_norm", c)
        for n in ("to_q", "to_k", "to_v", "to_out.0"):
            self._p(f"{name}.{n}.weight", (c, c), "rand")
            self._p(f"{name}.{n}.bias", (c,), "zeros")

    # -- forward ------------------------------------------------------------------------
    def _gn_silu(self, x, name):
        return F.silu(F.group_norm(x, self.cfg.norm_groups, self.w[name + ".weight"], self.w[name + ".bias"], eps=1e-6))

    def _c(self, x, name, pad=1):
        return F.conv2d(x, self.w[name + ".weight"], self.w[name + ".bias"], padding=pad)

    def _res(self, x, name, ci, co):
        h = self._c(self._gn_silu(x, name + ".norm1"), name + ".conv1")
        h = self._c(self._gn_silu(h, name + ".norm2"), name + ".conv2")
        if ci != co:
            x = self._c(x, name + ".conv_shortcut", pad=0)
        return x + h

    def _attention(self, x, name):
        b, c, hh, ww = x.shape
        h = F.group_norm(x, self.cfg.norm_groups, self.w[name + ".group_norm.weight"], self.w[name + ".group_norm.bias"], eps=1e-6)
        t = h.reshape(b, c, hh * ww).transpose(1, 2)
        lin = lambda n: F.linear(t, self.w[f"{name}.{n}.weight"].reshape(c, c), self.w[f"{name}.{n}.bias"])
        q, k, v = lin("to_q"), lin("to_k"), lin("to_v")
        o = F.scaled_dot_product_attention(q[:, None], k[:, None], v[:, None])[:, 0]
        o = F.linear(o, self.w[f"{name}.to_out.0.weight"].reshape(c, c), self.w[f"{name}.to_out.0.bias"])
        return x + o.transpose(1, 2).reshape(b, c, hh, ww)

    @torch.no_grad()
    def decode_tiled(self, latents: torch.Tensor, tile: int = 64, overlap: int = 16) -> torch.Tensor:
        """Decode in overlapping latent tiles of ``tile`` x ``tile`` and cross-fade the overlaps (linear
        ramps of ``overlap`` latent pixels), so that activation memory is bounded by the tile and not by
        the image. Tiles see only their own GroupNorm / attention context, so the result differs from
        :meth:`decode` by the usual tiling tolerance; images no larger than one tile take the plain path.
        (Reference: src/HartsyInference.Diffusion/Models/Vae/ tiled decode of its low-VRAM mode.)"""
        b, c, h, w = latents.shape
        if h <= tile and w <= tile:
            return self.decode(latents)
        f = 2 ** (len(self.cfg.block_out_channels) - 1)
        overlap = max(0, min(overlap, tile // 2))
        step = tile - overlap
        ys = list(range(0, max(h - overlap, 1), step))
        xs = list(range(0, max(w - overlap, 1), step))
        out = torch.zeros(b, 3, h * f, w * f)
        weight = torch.zeros(1, 1, h * f, w * f)
        for y0 in ys:
            for x0 in xs:
                y1, x1 = min(h, y0 + tile), min(w, x0 + tile)
                ya, xa = max(0, y1 - tile), max(0, x1 - tile)          # edge tiles keep the full tile size
                img = self.decode(latents[:, :, ya:y1, xa:x1]).cpu()
                th, tw = img.shape[-2], img.shape[-1]
                ramp = max(1, overlap * f)
                wy = torch.ones(th)
                wx = torch.ones(tw)
                if ya > 0:
                    wy[:ramp] = torch.linspace(0, 1, ramp + 2)[1:-1]
                if y1 < h:
                    wy[-ramp:] = torch.linspace(1, 0, ramp + 2)[1:-1]
                if xa > 0:
                    wx[:ramp] = torch.linspace(0, 1, ramp + 2)[1:-1]
                if x1 < w:
                    wx[-ramp:] = torch.linspace(1, 0, ramp + 2)[1:-1]
                m = (wy[:, None] * wx[None, :])[None, None]
                out[:, :, ya * f:y1 * f, xa * f:x1 * f] += img * m
                weight[:, :, ya * f:y1 * f, xa * f:x1 * f] += m
        return (out / weight.clamp_min(1e-6)).clamp(-1, 1)

    @torch.no_grad()
    def decode(self, latents: torch.Tensor) -> torch.Tensor:
        """latents [B, C, h, w] (model space) -> images [B, 3, 8h, 8w] in [-1, 1] (float32)."""
        z = latents.to(self.device).float() / self.cfg.scaling_factor + self.cfg.shift_factor
        x = self._c(z.to(self.dtype), "decoder.conv_in")
        top = self.cfg.block_out_channels[-1]
        x = self._res(x, "decoder.mid_block.resnets.0", top, top)
        x = self._attention(x, "decoder.mid_block.attentions.0")
        x = self._res(x, "decoder.mid_block.resnets.1", top, top)
        for blocks, up in self.up:
            for name, ci, co in blocks:
                x = self._res(x, name, ci, co)
            if up is not None:
                x = self._c(F.interpolate(x, scale_factor=2.0, mode="nearest"), up)
        x = self._c(self._gn_silu(x, "decoder.conv_norm_out"), "decoder.conv_out")
        return x.float().clamp(-1, 1)


class Vae2dEncoder(Vae2dDecoder):
    """The encoder half (image -> latent mean): conv_in, four down blocks of ResNets with a stride-2
    convolution between them (asymmetric right / bottom padding), the same mid block, GroupNorm +
    SiLU, conv_out to 2 x latent channels (mean | log-variance). Used by img2img and inpainting.
    Reference: src/HartsyInference.Diffusion/Models/Vae/ (VaeEncoder)."""

    def __init__(self, cfg: Vae2dConfig = FLUX_VAE, device="cpu", dtype=torch.bfloat16,
                 get: Optional[Callable[[str], Optional[torch.Tensor]]] = None, seed: int = 1):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        self._get = get
        self._g = torch.Generator().manual_seed(seed)
        self.w = {}
        ch = list(cfg.block_out_channels)
        self._conv("encoder.conv_in", ch[0], 3, 3)
        prev = ch[0]
        self.down: list[tuple[list[tuple[str, int, int]], Optional[str]]] = []
        for i, c in enumerate(ch):
            blocks = []
            for j in range(cfg.layers_per_block):
                name = f"encoder.down_blocks.{i}.resnets.{j}"
                self._resnet(name, prev, c)
                blocks.append((name, prev, c))
                prev = c
            dn = None
            if i < len(ch) - 1:
                dn = f"encoder.down_blocks.{i}.downsamplers.0.conv"
                self._conv(dn, c, c, 3)
            self.down.append((blocks, dn))
        self._resnet("encoder.mid_block.resnets.0", prev, prev)
        self._attn("encoder.mid_block.attentions.0", prev)
        self._resnet("encoder.mid_block.resnets.1", prev, prev)
        self._norm("encoder.conv_norm_out", prev)
        self._conv("encoder.conv_out", 2 * cfg.latent_channels, prev, 3)

    @torch.no_grad()
    def encode(self, images: torch.Tensor, sample: bool = False, generator: Optional[torch.Generator] = None) -> torch.Tensor:
        """images [B, 3, H, W] in [-1, 1] -> latents [B, C, H/8, W/8] in model space (fp32): the
        posterior mean (or a sample), shifted and scaled."""
        x = self._c(images.to(self.device).to(self.dtype), "encoder.conv_in")
        for blocks, dn in self.down:
            for name, ci, co in blocks:
                x = self._res(x, name, ci, co)
            if dn is not None:
                x = F.conv2d(F.pad(x, (0, 1, 0, 1)), self.w[dn + ".weight"], self.w[dn + ".bias"], stride=2)
        top = self.cfg.block_out_channels[-1]
        x = self._res(x, "encoder.mid_block.resnets.0", top, top)
        x = self._attention(x, "encoder.mid_block.attentions.0")
        x = self._res(x, "encoder.mid_block.resnets.1", top, top)
        moments = self._c(self._gn_silu(x, "encoder.conv_norm_out"), "encoder.conv_out").float()
        mean, logvar = moments.chunk(2, 1)
        z = mean
        if sample:
            std = torch.exp(0.5 * logvar.clamp(-30, 20))
            z = mean + std * torch.randn(mean.shape, generator=generator).to(mean.device)
        return (z - self.cfg.shift_factor) * self.cfg.scaling_factor

    def decode(self, latents):  # pragma: no cover - this half has no decoder weights
        raise NotImplementedError("Vae2dEncoder only encodes")


def to_rgb24(images: torch.Tensor) -> list[bytes]:
    """[B, 3, H, W] in [-1, 1] -> RGB24 byte strings."""
    u8 = ((images.float().clamp(-1, 1) + 1) * 127.5).round().to(torch.uint8).permute(0, 2, 3, 1).contiguous().cpu()
    return [u8[i].numpy().tobytes() for i in range(u8.shape[0])]
