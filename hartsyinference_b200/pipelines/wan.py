"""Wan text-to-video pipeline: umT5 encode -> noise -> N steps (cond + uncond DiT forwards, CFG
combine, UniPC or Euler update on the device) -> causal 3-D VAE decode -> frames.

Follows ``WanVideoPipeline.RunDenoise`` (src/HartsyInference.Video/Pipelines/WanVideoPipeline.cs:
191-543: CFG-parallel preload :251-274, context-parallel set-up :319-360, step loop :409-521, host
scheduler step :503). Parallel layouts: ``sp_comm`` = Ulysses group inside the transformer;
``cfg_comm`` = 2-rank communicator pairing a rank of the conditional group with its twin in the
unconditional group (CFG-parallel: each group runs one branch, the predictions are exchanged, both
groups apply the same update and stay in lock-step)."""
from __future__ import annotations

import time
import zlib
from dataclasses import dataclass
from typing import Callable, Optional

import torch

from .. import config, log
from ..engine.metrics import REGISTRY
from ..engine.requests import StepPreview, VideoGenerationResult, VideoRequest
from ..models.diffusion.schedulers import FlowMatchEulerScheduler, FlowUniPCScheduler
from ..models.dit.wan import WanTransformer
from ..models.vae.vae2d import to_rgb24
from ..models.vae.vae3d import Vae3dDecoder
from ..parallel.comm import Comm


@dataclass
class WanComponents:
    transformer: WanTransformer
    vae: Optional[Vae3dDecoder] = None
    text_encoder: Optional[object] = None
    tokenizer: Optional[object] = None


class WanPipeline:
    def __init__(self, comp: WanComponents, cfg_comm: Optional[Comm] = None):
        self.c = comp
        self.device = comp.transformer.device
        self.cfg_comm = cfg_comm
        self.last_step_ms: list[float] = []

    def encode_prompt(self, prompt: str) -> torch.Tensor:
        cfg = self.c.transformer.cfg
        if self.c.text_encoder is None or self.c.tokenizer is None:
            g = torch.Generator().manual_seed(zlib.crc32(prompt.encode("utf-8")) % (2 ** 31))
            return torch.randn(cfg.text_len, cfg.text_dim, generator=g)
        ids = torch.tensor(self.c.tokenizer.encode(prompt)[: cfg.text_len], dtype=torch.int64)
        ctx = self.c.text_encoder.encode(ids)
        if ctx.shape[0] < cfg.text_len:
            ctx = torch.cat([ctx, torch.zeros(cfg.text_len - ctx.shape[0], ctx.shape[1], dtype=ctx.dtype, device=ctx.device)])
        return ctx

    @torch.no_grad()
    def denoise(self, ctx: torch.Tensor, neg: Optional[torch.Tensor], frames: int, height: int, width: int, steps: int,
                cfg_scale: float, seed: int, scheduler: str = "unipc", shift: float = 5.0,
                on_step: Optional[Callable[[StepPreview], None]] = None) -> torch.Tensor:
        tr = self.c.transformer
        dev = self.device
        lt, lh, lw = (frames - 1) // 4 + 1, height // 8, width // 8
        g = torch.Generator().manual_seed(seed)
        x = torch.randn(tr.cfg.in_channels, lt, lh, lw, generator=g).to(dev)                # fp32
        c_pos = tr.encode_text(ctx.to(dev))
        c_neg = tr.encode_text(neg.to(dev)) if (neg is not None and cfg_scale != 1.0) else None
        uni = FlowUniPCScheduler(steps, shift=shift) if scheduler == "unipc" else None
        eul = FlowMatchEulerScheduler(steps, shift=shift) if uni is None else None
        branch = self.cfg_comm.rank if (self.cfg_comm is not None and self.cfg_comm.world == 2 and c_neg is not None) else None
        self.last_step_ms = []
        use_cuda = dev.type == "cuda"
        # the per-step scalars are staged in pinned host memory and copied as each step starts
        h_t = torch.tensor([float((uni or eul).timestep(i)) for i in range(steps)], dtype=torch.float32)
        if use_cuda:
            h_t = h_t.pin_memory()
        self.h2d_bytes_per_step = 4
        for i in range(steps):
            if use_cuda:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            t0 = time.perf_counter()
            t = h_t[i].to(dev, non_blocking=True)
            xin = x.to(torch.bfloat16)
            if branch is None:
                v = tr.forward(xin, t, c_pos)
                if c_neg is not None:
                    vu = tr.forward(xin, t, c_neg)
                    v = vu + cfg_scale * (v - vu)
            else:
                mine = tr.forward(xin, t, c_pos if branch == 0 else c_neg).contiguous()
                fused = self._cfg_kernel(mine.numel())
                if fused is not None:
                    v = fused.combine(mine.float(), cfg_scale)       # peer loads inside the combine kernel
                else:
                    both = self.cfg_comm.all_gather(mine[None], dim=0)
                    v = both[1] + cfg_scale * (both[0] - both[1])
            if uni is not None:
                x = uni.step(v, x)
            else:
                x = x + v.float() * eul.dt(i)
            if use_cuda:
                e1.record()
                e1.synchronize()
                ms = e0.elapsed_time(e1)
            else:
                ms = (time.perf_counter() - t0) * 1e3
            self.last_step_ms.append(ms)
            REGISTRY.set("hartsyinference_step_seconds", ms / 1e3, model="wan")
            if on_step is not None:
                on_step(StepPreview(i + 1, steps, latents=x))      # fp32 latents [C, T, H / 8, W / 8] on the device
        return x

    def _cfg_kernel(self, n: int):
        """The two-rank combine kernel over peer memory (parallel/cfg_combine.py), or None on CPU
        ranks, for sizes the kernel does not take, or when the peer mapping cannot be made."""
        if self.device.type != "cuda" or n % 8 != 0 or not config.get("fused_cfg_combine"):
            return None
        cur = getattr(self, "_cfg_fused", None)
        if cur is None or cur[0] < n:
            from ..parallel.cfg_combine import FusedCfgCombine
            try:
                if cur is not None and cur[1] is not None:
                    cur[1].close()
                self._cfg_fused = (n, FusedCfgCombine(self.cfg_comm, n, self.device))
                self.cfg_path = "peer loads inside the CFG combine kernel"
            except Exception as e:
                log.warn(f"[Collective] CFG combine kernel unavailable ({type(e).__name__}: {e}); using all_gather")
                self._cfg_fused = (1 << 62, None)
        return self._cfg_fused[1]

    def close(self) -> None:
        cur = getattr(self, "_cfg_fused", None)
        if cur is not None and cur[1] is not None:
            cur[1].close()
        self._cfg_fused = None

    def generate(self, req: VideoRequest, on_step: Optional[Callable[[StepPreview], None]] = None) -> VideoGenerationResult:
        seed = req.seed if req.seed is not None else int(time.time() * 1000) % (2 ** 31)
        ctx = self.encode_prompt(req.prompt)
        neg = self.encode_prompt(req.negative_prompt) if req.cfg_scale != 1.0 else None
        t0 = time.perf_counter()
        z = self.denoise(ctx, neg, req.frames, req.height, req.width, req.steps, req.cfg_scale, seed,
                         "unipc" if req.scheduler.startswith("uni") else "euler", req.shift, on_step)
        t_denoise = time.perf_counter() - t0
        frames: list[bytes] = []
        w = h = 0
        if self.c.vae is not None:
            vid = self.c.vae.decode(z[None])[0]                                             # [3, T, H, W]
            frames = to_rgb24(vid.permute(1, 0, 2, 3))
            h, w = vid.shape[-2], vid.shape[-1]
        log.info(f"[Wan] {req.width}x{req.height}x{req.frames}f {req.steps} steps in {t_denoise:.2f}s")
        return VideoGenerationResult(frames=frames, width=w, height=h, fps=req.fps, seed=seed,
                                     meta={"steps": req.steps, "denoise_s": t_denoise,
                                           "step_ms_median": sorted(self.last_step_ms)[len(self.last_step_ms) // 2] if self.last_step_ms else 0.0})
