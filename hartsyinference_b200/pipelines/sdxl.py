"""Stable Diffusion 1.5 and SDXL text-to-image pipelines: epsilon-prediction U-Net, Euler sampling over
the scaled-linear beta schedule, classifier-free guidance, 4-channel VAE.

Conditioning. SD 1.5: the final-norm token states of CLIP-L [77, 768]. SDXL: the second-to-last-layer
states of CLIP-L and CLIP-G side by side [77, 2048], the projected pooled CLIP-G vector [1280], and six
numbers (original size, crop offset, target size) that the U-Net codes with sinusoids. Conditional and
unconditional branches go through the U-Net as one batch of two; the guided prediction and the Euler
update are one fused kernel on the device (``ops.cfg_euler_step``). Without text encoders (synthetic
runs) the conditioning is deterministic noise derived from the prompt.

Reference: src/HartsyInference.Diffusion/Pipelines/StableDiffusion15Pipeline.cs, SdxlPipeline.cs.
"""
from __future__ import annotations

import time
import zlib
from dataclasses import dataclass
from typing import Callable, Optional

import torch

from .. import log, ops
from ..engine.requests import ImageRequest, ImageResult, StepPreview
from ..models.diffusion.schedulers import EulerDiscreteScheduler
from ..models.unet.unet2d import UNet2D
from ..models.vae.vae2d import Vae2dConfig, Vae2dDecoder, to_rgb24

SD15_VAE = Vae2dConfig(latent_channels=4, scaling_factor=0.18215, shift_factor=0.0)
SDXL_VAE = Vae2dConfig(latent_channels=4, scaling_factor=0.13025, shift_factor=0.0)


@dataclass
class SdComponents:
    unet: UNet2D
    vae: Optional[Vae2dDecoder] = None
    clip_l: Optional[Callable] = None        # prompt -> (token states [77, d], pooled [d])
    clip_g: Optional[Callable] = None        # SDXL only


class StableDiffusionPipeline:
    """SD 1.5 when the U-Net has no micro-conditioning, SDXL when it has."""

    def __init__(self, comp: SdComponents):
        self.c = comp
        self.device = comp.unet.device
        self.sdxl = comp.unet.cfg.addition_embed_dim > 0
        self.last_step_ms: list[float] = []

    def encode_prompt(self, prompt: str):
        """-> (context [77, cross_attention_dim], pooled [P] or None)."""
        c, cfg = self.c, self.c.unet.cfg
        pooled_dim = cfg.addition_embed_dim - 6 * cfg.addition_time_embed_dim if self.sdxl else 0
        if c.clip_l is None or (self.sdxl and c.clip_g is None):
            g = torch.Generator().manual_seed(zlib.crc32(("sd:" + prompt).encode("utf-8")) % (2 ** 31))
            return torch.randn(77, cfg.cross_attention_dim, generator=g), (torch.randn(pooled_dim, generator=g) if self.sdxl else None)
        sl, _ = c.clip_l(prompt)
        if not self.sdxl:
            return sl.float(), None
        sg, pg = c.clip_g(prompt)
        return torch.cat([sl.float(), sg.float()], -1), pg.float()

    @torch.no_grad()
    def denoise(self, cond, neg, height: int, width: int, steps: int, cfg_scale: float, seed: int,
                on_step: Optional[Callable[[StepPreview], None]] = None) -> torch.Tensor:
        unet, dev = self.c.unet, self.device
        sched = EulerDiscreteScheduler(steps)
        z = torch.randn(1, unet.cfg.in_channels, height // 8, width // 8, generator=torch.Generator().manual_seed(seed)).to(dev)
        z = z * sched.init_noise_sigma
        use_cfg = cfg_scale > 1.0 and neg is not None
        ctx = torch.stack([neg[0], cond[0]]) if use_cfg else cond[0][None]
        pooled = time_ids = None
        if self.sdxl:
            pooled = torch.stack([neg[1], cond[1]]) if use_cfg else cond[1][None]
            time_ids = torch.tensor([[height, width, 0, 0, height, width]], dtype=torch.float32).expand(ctx.shape[0], -1)
        self.last_step_ms = []
        for i in range(steps):
            t0 = time.perf_counter()
            xin = sched.scale_input(z, i)
            xin = torch.cat([xin, xin]) if use_cfg else xin
            eps = unet.forward(xin, sched.timesteps[i].expand(xin.shape[0]), ctx, pooled, time_ids)
            dt = float(sched.sigmas[i + 1] - sched.sigmas[i])
            if use_cfg:
                flat = z.reshape(-1).contiguous()
                ops.cfg_euler_step(flat, eps[1].reshape(-1).to(torch.bfloat16).contiguous(), eps[0].reshape(-1).to(torch.bfloat16).contiguous(),
                                   cfg_scale, dt)
                z = flat.reshape(z.shape)
            else:
                z = z + eps * dt
            if dev.type == "cuda":
                torch.cuda.synchronize(dev)
            self.last_step_ms.append((time.perf_counter() - t0) * 1e3)
            if on_step is not None:
                on_step(StepPreview(i + 1, steps))
        return z

    def generate(self, req: ImageRequest, on_step: Optional[Callable[[StepPreview], None]] = None) -> ImageResult:
        seed = req.seed if req.seed is not None else int(time.time() * 1000) % (2 ** 31)
        scale = req.cfg_scale if req.cfg_scale > 1.0 else req.guidance
        cond = self.encode_prompt(req.prompt)
        neg = self.encode_prompt(req.negative_prompt or "") if scale > 1.0 else None
        t0 = time.perf_counter()
        z = self.denoise(cond, neg, req.height, req.width, req.steps, scale, seed, on_step)
        t_denoise = time.perf_counter() - t0
        img = self.c.vae.decode(z) if self.c.vae is not None else torch.zeros(1, 3, req.height, req.width)
        log.info(f"[{'SDXL' if self.sdxl else 'SD1.5'}] {req.width}x{req.height} {req.steps} steps in {t_denoise:.2f}s")
        return ImageResult(rgb=to_rgb24(img)[0], width=img.shape[-1], height=img.shape[-2], seed=seed,
                           meta={"steps": req.steps, "denoise_s": t_denoise, "cfg_scale": scale, "scheduler": "euler_discrete"})
