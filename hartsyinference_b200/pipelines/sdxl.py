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
    controlnet: Optional[object] = None      # models.unet.unet2d.ControlNet of the same family
    image_projector: Optional[Callable] = None   # install_ip_adapter's projector: CLIP image embedding -> image tokens
    image_encoder: Optional[Callable] = None     # picture -> CLIP image embedding [1, E]


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
                on_step: Optional[Callable[[StepPreview], None]] = None, control: Optional[torch.Tensor] = None,
                control_scale: float = 1.0, image_embeds: Optional[torch.Tensor] = None, image_scale: float = 1.0) -> torch.Tensor:
        """``control`` [1, 3, height, width] in [0, 1] drives the ControlNet (both guidance branches see it);
        ``image_embeds`` [1, E] is the picture prompt: its tokens go to the conditional branch, zeros' tokens to the
        unconditional one."""
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
        if control is not None and self.c.controlnet is None:
            raise ValueError("a control image was given but no ControlNet is loaded beside the model")
        tokens = None
        if image_embeds is not None:
            if self.c.image_projector is None:
                raise ValueError("a picture prompt was given but no image adapter is loaded beside the model")
            tokens = self.c.image_projector(image_embeds)
            if use_cfg:
                tokens = torch.cat([self.c.image_projector(torch.zeros_like(image_embeds)), tokens])
        self.last_step_ms = []
        for i in range(steps):
            t0 = time.perf_counter()
            xin = sched.scale_input(z, i)
            xin = torch.cat([xin, xin]) if use_cfg else xin
            ts = sched.timesteps[i].expand(xin.shape[0])
            down = mid = None
            if control is not None:
                down, mid = self.c.controlnet.forward(xin, ts, ctx, control.expand(xin.shape[0], -1, -1, -1), pooled, time_ids, control_scale)
            eps = unet.forward(xin, ts, ctx, pooled, time_ids, down, mid, tokens, image_scale)
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

    @staticmethod
    def _picture(image, height: int, width: int) -> torch.Tensor:
        """Path / PIL image / HWC or CHW tensor -> [1, 3, height, width] in [0, 1]."""
        import numpy as np
        if isinstance(image, (str, bytes)) or hasattr(image, "__fspath__"):
            from PIL import Image
            image = Image.open(image)
        if hasattr(image, "convert"):
            image = torch.from_numpy(np.asarray(image.convert("RGB")).copy())
        t = torch.as_tensor(image)
        if t.dtype == torch.uint8:
            t = t.float() / 255.0
        if t.ndim == 3 and t.shape[-1] == 3 and t.shape[0] != 3:
            t = t.permute(2, 0, 1)
        t = t.float()[None] if t.ndim == 3 else t.float()
        if t.shape[-2:] != (height, width):
            t = torch.nn.functional.interpolate(t, size=(height, width), mode="bilinear", align_corners=False)
        return t.clamp(0, 1)

    def generate(self, req: ImageRequest, on_step: Optional[Callable[[StepPreview], None]] = None) -> ImageResult:
        seed = req.seed if req.seed is not None else int(time.time() * 1000) % (2 ** 31)
        scale = req.cfg_scale if req.cfg_scale > 1.0 else req.guidance
        cond = self.encode_prompt(req.prompt)
        neg = self.encode_prompt(req.negative_prompt or "") if scale > 1.0 else None
        t0 = time.perf_counter()
        control = embeds = None
        if getattr(req, "control_image", None) is not None:
            control = self._picture(req.control_image, req.height, req.width)
        if getattr(req, "image_prompt", None) is not None:
            if self.c.image_encoder is None:
                raise ValueError("a picture prompt was given but no image encoder is loaded beside the model")
            embeds = self.c.image_encoder(req.image_prompt)
        z = self.denoise(cond, neg, req.height, req.width, req.steps, scale, seed, on_step, control,
                         float(getattr(req, "control_strength", 1.0) or 1.0), embeds, float(getattr(req, "image_prompt_scale", 1.0) or 1.0))
        t_denoise = time.perf_counter() - t0
        img = self.c.vae.decode(z) if self.c.vae is not None else torch.zeros(1, 3, req.height, req.width)
        log.info(f"[{'SDXL' if self.sdxl else 'SD1.5'}] {req.width}x{req.height} {req.steps} steps in {t_denoise:.2f}s")
        return ImageResult(rgb=to_rgb24(img)[0], width=img.shape[-1], height=img.shape[-2], seed=seed,
                           meta={"steps": req.steps, "denoise_s": t_denoise, "cfg_scale": scale, "scheduler": "euler_discrete"})
