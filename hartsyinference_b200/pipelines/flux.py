"""Flux text-to-image pipeline: text encode -> noise -> pack 2x2 -> N denoise steps (DiT forward +
fused CFG / Euler step on the device) -> unpack -> VAE decode -> RGB24.

Follows ``FluxPipeline`` (src/HartsyInference.Diffusion/Pipelines/FluxPipeline.cs: denoise loop
:722-1002, CFG-parallel branch :750-807, fused CfgEulerStep :821) with the FlowMatch-Euler schedule
and Flux's dynamic shift. True CFG (``cfg_scale > 1``) runs a second, unconditional forward, or,
with ``cfg_comm`` (two ranks / two groups), one branch per group whose outputs are exchanged
before the combine + step kernel. A first-block cache (relative-L1 on the timestep embedding's
modulated input, as ``DeviceFeatureCache``: ShouldCompute:82) can skip the transformer on steps
whose conditioning changed little.
"""
from __future__ import annotations

import time
import zlib
from dataclasses import dataclass
from typing import Callable, Optional

import torch

from .. import log
from ..engine.metrics import REGISTRY
from ..engine.requests import ImageRequest, ImageResult, StepPreview
from ..models.diffusion.preview import in_guidance_interval
from ..models.diffusion.schedulers import FlowMatchEulerScheduler, flux_mu
from ..models.dit.flux import FluxTransformer, flux_ids
from ..models.vae.vae2d import Vae2dDecoder, to_rgb24
from ..parallel.comm import Comm


def pack_latents(z: torch.Tensor) -> torch.Tensor:
    """[B, C, H, W] -> [B, (H/2)(W/2), 4C] (2x2 patches, channel-major inside a patch)."""
    b, c, h, w = z.shape
    return z.reshape(b, c, h // 2, 2, w // 2, 2).permute(0, 2, 4, 1, 3, 5).reshape(b, (h // 2) * (w // 2), c * 4)


def unpack_latents(x: torch.Tensor, h: int, w: int) -> torch.Tensor:
    b, _, c4 = x.shape
    c = c4 // 4
    return x.reshape(b, h // 2, w // 2, c, 2, 2).permute(0, 3, 1, 4, 2, 5).reshape(b, c, h, w)


@dataclass
class FluxComponents:
    transformer: FluxTransformer
    vae: Optional[Vae2dDecoder] = None
    t5: Optional[object] = None
    clip: Optional[object] = None
    vae_encoder: Optional[object] = None      # Vae2dEncoder: img2img / inpainting start from an encoded image
    controlnet: Optional[object] = None       # FluxControlNet: residuals from a control image's latents
    t5_tokenizer: Optional[object] = None
    clip_tokenizer: Optional[object] = None
    redux: Optional[object] = None            # models.dit.redux.ReduxImageEncoder
    image_states: Optional[Callable] = None   # picture -> SigLIP patch states [n, 1152]


class FluxPipeline:
    def __init__(self, comp: FluxComponents, cfg_comm: Optional[Comm] = None):
        self.c = comp
        self.device = comp.transformer.device
        self.cfg_comm = cfg_comm            # 2-rank communicator pairing the cond / uncond branches
        self.last_step_ms: list[float] = []

    # -- conditioning -------------------------------------------------------------------
    def encode_prompt(self, prompt: str, max_len: int = 512) -> tuple[torch.Tensor, torch.Tensor]:
        c = self.c
        tdim, pdim = c.transformer.cfg.context_dim, c.transformer.cfg.pooled_dim
        if c.t5 is None or c.t5_tokenizer is None:
            # synthetic conditioning (no text encoder loaded): deterministic N(0, 1) from the prompt text
            g = torch.Generator().manual_seed(zlib.crc32(prompt.encode("utf-8")) % (2 ** 31))
            return torch.randn(max_len, tdim, generator=g), torch.randn(pdim, generator=g)
        from ..models.diffusion.prompt_weighting import apply_token_weights, parse_prompt_weights, token_weights
        runs = parse_prompt_weights(prompt)
        prompt = "".join(t for t, _ in runs)            # the text without the weighting syntax
        weights: list[float] = []
        if len(runs) > 1 or runs[0][1] != 1.0:
            # weighted prompt: tokenise run by run so every token knows its weight; the encoders see the plain text
            tok = c.t5_tokenizer
            piece_ids, weights = token_weights(runs, lambda t: tok.encode(t, add_special=False), max_len - 1)
            eos = tok.encode("", add_special=True)
            ids = torch.tensor(piece_ids + eos, dtype=torch.int64)
        else:
            ids = torch.tensor(c.t5_tokenizer.encode(prompt)[:max_len], dtype=torch.int64)
        ctx = c.t5.encode(ids)
        if weights:
            ctx = apply_token_weights(ctx, weights)
        if ctx.shape[0] < max_len:
            ctx = torch.cat([ctx, torch.zeros(max_len - ctx.shape[0], ctx.shape[1], dtype=ctx.dtype, device=ctx.device)])
        pooled = torch.zeros(pdim)
        if c.clip is not None and c.clip_tokenizer is not None:
            cid = torch.tensor(c.clip_tokenizer.encode(prompt)[:77], dtype=torch.int64)
            pooled = c.clip.encode(cid)[1]
        return ctx, pooled

    # -- denoise ------------------------------------------------------------------------
    @torch.no_grad()
    def denoise(self, ctx: torch.Tensor, pooled: torch.Tensor, height: int, width: int, steps: int, guidance: float,
                seed: int, neg: Optional[tuple[torch.Tensor, torch.Tensor]] = None, cfg_scale: float = 1.0,
                on_step: Optional[Callable[[StepPreview], None]] = None, step_cache_threshold: float = 0.0, first_block_cache: float = 0.0,
                latents: Optional[torch.Tensor] = None, init_latents: Optional[torch.Tensor] = None, strength: float = 1.0,
                mask: Optional[torch.Tensor] = None, control_latents: Optional[torch.Tensor] = None,
                control_strength: float = 1.0, channel_cond: Optional[torch.Tensor] = None,
                guidance_interval: Optional[tuple] = None, cfg_renorm_min: Optional[float] = None,
                cfg_row_norm: bool = False) -> torch.Tensor:
        """Returns the final latents [1, C, H/8, W/8] fp32 on the device.

        ``guidance_interval`` (start, end) limits true classifier-free guidance to the steps inside it
        (single-process runs; with the two branches on two ranks both always run).

        ``init_latents`` [1, C, H/8, W/8] with ``strength`` < 1 starts from the image noised to the
        sigma of step ``steps * (1 - strength)`` and runs the remaining steps (img2img). ``mask``
        [1, 1, H/8, W/8] (1 = repaint) additionally pins the unmasked region to the original image,
        re-noised to each step's sigma (inpainting)."""
        tr = self.c.transformer
        dev = self.device
        C = tr.cfg.latent_channels // 4
        lh, lw = height // 8, width // 8
        g = torch.Generator().manual_seed(seed)
        z = latents if latents is not None else torch.randn(1, C, lh, lw, generator=g)
        x = pack_latents(z.float()).to(dev).contiguous()                           # [1, S, 4C] fp32
        S = x.shape[1]
        img_ids, txt_ids = flux_ids(lh // 2, lw // 2, ctx.shape[0], dev)
        sched = FlowMatchEulerScheduler(steps, mu=flux_mu(S))
        extra_packed = None
        if tr.cfg.in_channels != tr.cfg.latent_channels:
            if channel_cond is None or channel_cond.shape[2] != tr.cfg.in_channels - tr.cfg.latent_channels:
                raise ValueError(f"this transformer reads {tr.cfg.in_channels - tr.cfg.latent_channels} conditioning channels "
                                 "per token beside the latents (a control image, or image + mask for the Fill variant)")
            extra_packed = channel_cond.to(dev).to(torch.bfloat16).contiguous()
        ctrl_packed = None
        if control_latents is not None and self.c.controlnet is not None:
            ctrl_packed = pack_latents(control_latents.float()).to(dev).to(torch.bfloat16).contiguous()
        first_step = 0
        init_packed = noise_packed = mask_packed = None
        if init_latents is not None:
            first_step = min(steps - 1, max(0, int(round(steps * (1.0 - strength))))) if strength < 1.0 else 0
            init_packed = pack_latents(init_latents.float()).to(dev).contiguous()
            noise_packed = x.clone()
            s0 = sched.sigma(first_step)
            x = (s0 * noise_packed + (1.0 - s0) * init_packed).contiguous()      # flow matching: x_t = t noise + (1 - t) x_0
            if mask is not None:
                mask_packed = pack_latents(mask.float().expand(1, C, lh, lw)).to(dev).contiguous()
        ctx_d, pooled_d = ctx.to(dev)[None], pooled.to(dev)[None]
        gvec = torch.tensor([guidance], device=dev) if tr.cfg.guidance_embed else None
        true_cfg = cfg_scale > 1.0 and neg is not None
        branch = None
        if true_cfg and self.cfg_comm is not None and self.cfg_comm.world == 2:
            branch = self.cfg_comm.rank                                           # 0 = cond, 1 = uncond
        # fused peer-memory combine + Euler step (one kernel, no all_gather) when the two branches sit
        # on GPUs that can map each other's memory; the step cache needs the combined velocity, so it
        # keeps the all_gather path
        fused_cfg = None
        if branch is not None and dev.type == "cuda" and step_cache_threshold <= 0 and S * x.shape[2] % 8 == 0:
            from .. import config as _config
            if _config.get("fused_comm") and not _config.get("p2p_disable"):
                fused_cfg = self._fused_cfg(S * x.shape[2], dev)
        cache_prev_t: Optional[torch.Tensor] = None
        cache_v: Optional[torch.Tensor] = None
        # first-block cache: one per CFG branch, decided inside the transformer after block 0
        from ..models.dit.step_cache import FirstBlockCache
        fbc = [FirstBlockCache(first_block_cache), FirstBlockCache(first_block_cache)] if first_block_cache > 0 else [None, None]
        self.last_step_ms = []
        use_cuda = dev.type == "cuda"
        # the per-step scalars are staged in pinned host memory and copied as each step starts
        h_sigmas = torch.tensor([sched.sigma(i) for i in range(steps)], dtype=torch.float32)
        if use_cuda:
            h_sigmas = h_sigmas.pin_memory()
        self.h2d_bytes_per_step = 4
        for i in range(first_step, steps):
            if use_cuda:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            t0 = time.perf_counter()
            sigma = h_sigmas[i:i + 1].to(dev, non_blocking=True)
            skip = False
            if step_cache_threshold > 0 and cache_v is not None:
                temb = tr.time_embedding(sigma, gvec, pooled_d).float()
                rel = ((temb - cache_prev_t).abs().mean() / cache_prev_t.abs().mean().clamp_min(1e-6)).item()
                skip = rel < step_cache_threshold
            if skip:
                v_cond, v_unc = cache_v, None
            else:
                xin = x.to(torch.bfloat16)
                if extra_packed is not None:      # Canny / Depth / Fill variants: conditioning rides along channel-wise
                    xin = torch.cat([xin, extra_packed], 2)
                ctl = None
                if ctrl_packed is not None:      # the ControlNet branch sees the conditional prompt
                    ctl = self.c.controlnet.residuals(xin, ctrl_packed, ctx_d, sigma, pooled_d, img_ids, txt_ids, gvec, control_strength)
                if branch is None:
                    v_cond = tr.forward(xin, ctx_d, sigma, pooled_d, img_ids, txt_ids, gvec, step_cache=fbc[0], control=ctl)
                    v_unc = tr.forward(xin, neg[0].to(dev)[None], sigma, neg[1].to(dev)[None], img_ids, txt_ids, gvec,
                                       step_cache=fbc[1]) if (true_cfg and in_guidance_interval(i, steps, guidance_interval)) else None
                else:
                    c_in, p_in = (ctx_d, pooled_d) if branch == 0 else (neg[0].to(dev)[None], neg[1].to(dev)[None])
                    mine = tr.forward(xin, c_in, sigma, p_in, img_ids, txt_ids, gvec, step_cache=fbc[0],
                                      control=ctl if branch == 0 else None).contiguous()
                    if fused_cfg is not None:
                        fused_cfg.step(x, mine, cfg_scale, sched.dt(i))
                        v_cond = None
                    else:
                        both = self.cfg_comm.all_gather(mine[None], dim=0)         # [2, 1, S, C]
                        v_cond, v_unc = both[0].contiguous(), both[1].contiguous()
                if step_cache_threshold > 0:
                    cache_prev_t = tr.time_embedding(sigma, gvec, pooled_d).float()
                    cache_v = v_cond if (not true_cfg or v_unc is None) else (cfg_scale * v_cond.float() + (1 - cfg_scale) * v_unc.float()).to(torch.bfloat16)
                    if true_cfg:
                        v_cond, v_unc = cache_v, None
            if v_cond is not None:
                sched.step(x, v_cond.contiguous(), i, v_unc, cfg_scale, renorm_min=cfg_renorm_min, row_norm=cfg_row_norm)
            if mask_packed is not None:
                # outside the mask the latent follows the original image at the next step's noise level
                s_next = sched.sigma(i + 1) if i + 1 < steps else 0.0
                known = s_next * noise_packed + (1.0 - s_next) * init_packed
                x.copy_(mask_packed * x + (1.0 - mask_packed) * known)
            if use_cuda:
                e1.record()
                e1.synchronize()
                ms = e0.elapsed_time(e1)
            else:
                ms = (time.perf_counter() - t0) * 1e3
            self.last_step_ms.append(ms)
            REGISTRY.set("hartsyinference_step_seconds", ms / 1e3, model="flux")
            if on_step is not None:
                on_step(StepPreview(i + 1, steps, latents=x))      # packed fp32 latents [1, S, 4C] on the device
        return unpack_latents(x, lh, lw)

    def _fused_cfg(self, elems: int, dev):
        """The fused CFG combine for latents of ``elems`` values (built once; None when the peer's
        memory cannot be mapped)."""
        cur = getattr(self, "_fused_cfg_obj", None)
        if cur is not None and cur.max_elems >= elems:
            return cur
        try:
            from ..parallel.cfg_combine import FusedCfgCombine
            self._fused_cfg_obj = FusedCfgCombine(self.cfg_comm, elems, dev)
        except Exception as e:      # no peer access: keep the all_gather path
            from .. import log
            log.decision("Collective", f"fused CFG combine unavailable ({type(e).__name__}: {e}); using all_gather")
            self._fused_cfg_obj = None
        return self._fused_cfg_obj

    def _channel_conditioning(self, req: ImageRequest) -> torch.Tensor:
        """Packed per-token conditioning [1, S, extra] for the channel-concatenation variants:
        Canny / Depth = the control image's latents; Fill = the masked image's latents and the mask
        folded 8 x 8 into channels (then packed 2 x 2 like the latents)."""
        tcfg = self.c.transformer.cfg
        extra = tcfg.in_channels - tcfg.latent_channels
        if self.c.vae_encoder is None:
            raise ValueError("this variant needs the VAE encoder to embed its conditioning image")
        h, w = req.height, req.width
        if extra == tcfg.latent_channels:                    # control image only
            if req.control_image is None:
                raise ValueError("this model needs ImageRequest.control_image")
            return pack_latents(self.c.vae_encoder.encode(self._image_tensor(req.control_image, w, h)).float())
        if req.init_image is None or req.mask_image is None:
            raise ValueError("the Fill variant needs ImageRequest.init_image and mask_image")
        img = self._image_tensor(req.init_image, w, h)
        m = (self._image_tensor(req.mask_image, w, h)[:, :1] * 0.5 + 0.5 > 0.5).float()
        lat = pack_latents(self.c.vae_encoder.encode(img * (1 - m)).float())
        folded = m.reshape(1, h // 8, 8, w // 8, 8).permute(0, 2, 4, 1, 3).reshape(1, 64, h // 8, w // 8)
        return torch.cat([lat, pack_latents(folded).to(lat.device)], 2)

    @staticmethod
    def _image_tensor(image, width: int, height: int) -> torch.Tensor:
        """Path, PIL image, uint8 HWC array / tensor or float CHW tensor in [0, 1] -> [1, 3, height, width] in [-1, 1]."""
        if isinstance(image, (str, bytes)) or hasattr(image, "__fspath__"):
            from PIL import Image
            image = Image.open(image)
        if hasattr(image, "convert"):
            import numpy as np
            image = torch.from_numpy(np.asarray(image.convert("RGB")).copy())
        t = torch.as_tensor(image)
        if t.dtype == torch.uint8:
            t = t.float() / 255.0
        if t.ndim == 2:
            t = t[None].expand(3, -1, -1)
        if t.ndim == 3 and t.shape[-1] in (1, 3) and t.shape[0] not in (1, 3):
            t = t.permute(2, 0, 1)
        if t.shape[0] == 1:
            t = t.expand(3, -1, -1)
        t = t.float()[None]
        if t.shape[-2:] != (height, width):
            t = torch.nn.functional.interpolate(t, size=(height, width), mode="bilinear", align_corners=False, antialias=True)
        return t.clamp(0, 1) * 2.0 - 1.0

    def _with_previews(self, on_step, req):
        """Wrap the step callback so that every ``req.preview_every``-th step carries an RGB preview of the
        latents (a linear map fitted once against this pipeline's VAE)."""
        every = int(getattr(req, "preview_every", 0) or 0)
        if on_step is None or every <= 0 or self.c.vae is None:
            return on_step
        if getattr(self, "_previewer", None) is None:
            from ..models.diffusion.preview import LatentPreviewer
            self._previewer = LatentPreviewer.fit(self.c.vae, self.c.transformer.cfg.latent_channels // 4)
        lh, lw = req.height // 8, req.width // 8

        def wrapped(p: StepPreview):
            if p.step % every == 0 and p.latents is not None:
                p.preview_rgb, p.preview_width, p.preview_height = self._previewer.rgb(unpack_latents(p.latents, lh, lw))
            on_step(p)
        return wrapped

    def generate(self, req: ImageRequest, on_step: Optional[Callable[[StepPreview], None]] = None) -> ImageResult:
        seed = req.seed if req.seed is not None else int(time.time() * 1000) % (2 ** 31)
        ctx, pooled = self.encode_prompt(req.prompt)
        neg = self.encode_prompt(req.negative_prompt) if req.cfg_scale > 1.0 else None
        if getattr(req, "image_prompt", None) is not None:
            if self.c.redux is None or self.c.image_states is None:
                raise ValueError("a picture prompt needs the Redux projector and its image encoder beside the model")
            tokens = self.c.redux(self.c.image_states(req.image_prompt), float(getattr(req, "image_prompt_scale", 1.0)))
            ctx = torch.cat([ctx.to(tokens.device), tokens.to(ctx.dtype)], 0)
            if neg is not None:                   # the unconditional branch sees as many (empty) picture tokens
                neg = (torch.cat([neg[0].to(tokens.device), torch.zeros_like(tokens).to(neg[0].dtype)], 0), neg[1])
        t0 = time.perf_counter()
        init_latents = mask = None
        if req.init_image is not None:
            if self.c.vae_encoder is None:
                raise ValueError("img2img / inpainting needs the VAE encoder (FluxComponents.vae_encoder)")
            init_latents = self.c.vae_encoder.encode(self._image_tensor(req.init_image, req.width, req.height))
            if getattr(req, "mask_image", None) is not None:
                m = self._image_tensor(req.mask_image, req.width, req.height)[:, :1] * 0.5 + 0.5
                mask = (torch.nn.functional.interpolate(m, size=(req.height // 8, req.width // 8), mode="area") > 0.5).float()
        control_latents = channel_cond = None
        tcfg = self.c.transformer.cfg
        if tcfg.in_channels != tcfg.latent_channels:
            channel_cond = self._channel_conditioning(req)
        elif getattr(req, "control_image", None) is not None:
            if self.c.controlnet is None or self.c.vae_encoder is None:
                raise ValueError("a control image needs a ControlNet and the VAE encoder (FluxComponents.controlnet / vae_encoder)")
            control_latents = self.c.vae_encoder.encode(self._image_tensor(req.control_image, req.width, req.height))
        on_step = self._with_previews(on_step, req)
        z = self.denoise(ctx, pooled, req.height, req.width, req.steps, req.guidance, seed, neg, req.cfg_scale, on_step,
                         req.step_cache_threshold, init_latents=init_latents, strength=req.strength, mask=mask,
                         control_latents=control_latents, control_strength=getattr(req, "control_strength", 1.0),
                         channel_cond=channel_cond, guidance_interval=getattr(req, "guidance_interval", None),
                         cfg_renorm_min=getattr(req, "cfg_renorm_min", None), cfg_row_norm=bool(getattr(req, "cfg_row_norm", False)))
        t_denoise = time.perf_counter() - t0
        if self.c.vae is None:
            img = torch.zeros(1, 3, req.height, req.width)
        elif getattr(req, "vae_tile", 0) > 0:
            img = self.c.vae.decode_tiled(z, req.vae_tile, req.vae_tile // 4)
        else:
            img = self.c.vae.decode(z)
        rgb = to_rgb24(img)[0]
        meta = {"steps": req.steps, "denoise_s": t_denoise, "step_ms_median": sorted(self.last_step_ms)[len(self.last_step_ms) // 2] if self.last_step_ms else 0.0,
                "sampler": "euler", "scheduler": "flow_match_euler", "guidance": req.guidance}
        log.info(f"[Flux] {req.width}x{req.height} {req.steps} steps in {t_denoise:.2f}s")
        return ImageResult(rgb=rgb, width=img.shape[-1], height=img.shape[-2], seed=seed, meta=meta)
