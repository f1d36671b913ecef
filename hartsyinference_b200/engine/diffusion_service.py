"""Image and video services: resolve a model spec to a pipeline (cached per placement), run it.

Counterparts: ``ImagesService.GenerateAsync`` (src/HartsyInference.Engine/Services/ImagesService.cs:
26-52), the video service, and the per-family recipes that wire DiT + text encoders + VAE
(src/HartsyInference.Engine/Recipes/Image/Flux1Recipe*.cs, Recipes/Video/). A spec whose
``requested`` is ``synthetic:<family>[-tiny]`` builds a random-init model of that architecture
(benchmarks and tests; there are no real checkpoints on an offline machine)."""
from __future__ import annotations

from pathlib import Path
from typing import Callable, Optional

import torch

from .. import config, log
from ..assets.safetensors import ShardedCheckpoint
from ..exceptions import UnsupportedModelError
from .recipes import IMAGE_RECIPES, VIDEO_RECIPES, RecipeContext, load_clip_text as _load_clip_text, load_t5 as _load_t5, with_loras as _with_loras  # noqa: F401
from .requests import EngineOptions, ImageRequest, ImageResult, ModelSpec, StepPreview, VideoGenerationResult, VideoRequest


class _PipelineCache:
    """Pipelines cached per (model, placement, device). ``ranks`` (see :mod:`.distributed`) makes the
    service SPMD: rank 0's ``generate`` is first broadcast as a command so that every rank runs the
    same denoise loop and the collectives inside the transformer / the CFG exchange line up; the
    placement's tensor- or sequence-parallel group goes to the transformer, its CFG pair to the
    pipeline. Without ``ranks`` the placement's ``text_encoder_device`` / ``vae_device`` ordinals put
    those components on other GPUs of the same process (the reference's component placement,
    src/HartsyInference.Core/Backends/PlacementConfig.cs:23,26)."""
    COMMAND = ""

    def __init__(self, options: EngineOptions, device: str, ranks=None):
        self.options, self.device = options, device
        self.ranks = ranks
        self._pipes: dict[str, object] = {}
        self._progress = None
        if ranks is not None and self.COMMAND:
            ranks.register(self.COMMAND, self._generate_local)

    def _comms(self):
        """(inner group, CFG pair) of this rank for the engine's placement; (None, None) single process."""
        if self.ranks is None:
            return None, None
        g = self.ranks.groups(self.options.placement)
        return (g.inner if g.inner.world > 1 else None), g.cfg

    def _component_device(self, ordinal: int) -> str:
        """Device of a text encoder / VAE: the placement's ordinal when one is given (single process,
        CUDA), else the denoiser's device."""
        if ordinal is None or ordinal < 0 or self.ranks is not None or not self.device.startswith("cuda"):
            return self.device
        if ordinal >= torch.cuda.device_count():
            raise UnsupportedModelError(f"placement names cuda:{ordinal}, {torch.cuda.device_count()} device(s) are visible")
        log.decision("Placement", f"component on cuda:{ordinal} (denoiser on {self.device})")
        return f"cuda:{ordinal}"

    def _context(self, spec: ModelSpec, loras: tuple = ()) -> RecipeContext:
        """Everything a recipe needs: checkpoint (None for ``synthetic:`` specs), devices and groups."""
        fp8 = bool(config.get("fp8_linears")) and self.device.startswith("cuda")
        inner, cfg_comm = self._comms()
        pl = self.options.placement
        ctx = RecipeContext(spec, self.device, self.options, fp8, inner, cfg_comm,
                            self._component_device(pl.text_encoder_device), self._component_device(pl.vae_device), loras)
        if not spec.requested.startswith("synthetic:"):
            path = Path(spec.local_path or spec.requested)
            if not path.exists():
                raise UnsupportedModelError(f"{spec.requested}: no such checkpoint")
            ctx.root = path
            # a diffusers-layout directory keeps the transformer, VAE, encoders and tokenizers in sub-folders
            sub = next((path / n for n in ("transformer", "unet") if (path / n).exists()), path)
            ctx.checkpoint = ShardedCheckpoint(sub)
        return ctx

    def generate(self, spec: ModelSpec, req, progress=None):
        if self.ranks is None:
            return self._generate_local(spec, req, progress)
        self._progress = progress            # callbacks stay on rank 0
        try:
            return self.ranks.command(self.COMMAND, spec, req)
        finally:
            self._progress = None

    def key(self, spec: ModelSpec, loras: tuple = ()) -> str:
        tag = "|".join(f"{p}@{s:g}" for p, s in loras)
        return f"{spec.local_path or spec.requested}|{self.options.placement.cache_key}|{self.device}" + (f"|lora:{tag}" if tag else "")

    def loaded_keys(self) -> list[str]:
        return list(self._pipes)

    def release(self, key: Optional[str] = None) -> None:
        self._release_local(key)

    def _release_local(self, key: Optional[str] = None) -> None:
        if key is None:
            self._pipes.clear()
        else:
            self._pipes.pop(key, None)
        if torch.cuda.is_available():
            torch.cuda.empty_cache()


def apply_recipe_defaults(spec: ModelSpec, req, recipe=None):
    """Fields the caller left at the request type's own default take the catalog entry's value for the
    model (steps, guidance, size, frames), else the family recipe's (engine/recipes.py)."""
    if not spec.catalog:
        return recipe.defaults.apply(req) if recipe is not None and not spec.requested.startswith("synthetic:") else req
    import dataclasses
    from ..assets.catalog import ModelCatalog
    entry = ModelCatalog().find(spec.catalog)
    if entry is None or not entry.defaults:
        return req
    changes = {}
    for f in dataclasses.fields(req):
        if f.name in entry.defaults and getattr(req, f.name) == f.default:
            changes[f.name] = entry.defaults[f.name]
    return dataclasses.replace(req, **changes) if changes else req


class ImagesService(_PipelineCache):
    COMMAND = "images.generate"

    def _build(self, spec: ModelSpec, loras: tuple = ()):
        ctx = self._context(spec, loras)
        recipe = IMAGE_RECIPES.resolve(spec, ctx.checkpoint)
        pipe = recipe.construct(ctx)
        pipe.recipe = recipe
        return pipe

    def pipeline(self, spec: ModelSpec, loras: tuple = ()):
        k = self.key(spec, loras)
        if k not in self._pipes:
            log.info(f"[Images] constructing pipeline for {spec.requested}" + (f" with {len(loras)} LoRA adapter(s)" if loras else ""))
            self._pipes[k] = self._build(spec, loras)
        return self._pipes[k]

    def _generate_local(self, spec: ModelSpec, req: ImageRequest, progress: Optional[Callable[[StepPreview], None]] = None) -> ImageResult:
        loras = tuple((str(p), float(s)) for p, s in (req.loras or ()))
        if loras and spec.requested.startswith("synthetic:"):
            raise UnsupportedModelError("LoRA adapters need a checkpoint to merge into")
        if req.seed is None and self.ranks is not None:
            raise ValueError("a multi-process engine needs ImageRequest.seed (every rank must draw the same noise)")
        pipe = self.pipeline(spec, loras)
        pipe.recipe.check_request(req)
        return pipe.generate(apply_recipe_defaults(spec, req, pipe.recipe), progress or self._progress)


class VideoService(_PipelineCache):
    COMMAND = "video.generate"

    def _build(self, spec: ModelSpec):
        ctx = self._context(spec)
        recipe = VIDEO_RECIPES.resolve(spec, ctx.checkpoint)
        pipe = recipe.construct(ctx)
        pipe.recipe = recipe
        return pipe

    def pipeline(self, spec: ModelSpec):
        k = self.key(spec)
        if k not in self._pipes:
            log.info(f"[Video] constructing pipeline for {spec.requested}")
            self._pipes[k] = self._build(spec)
        return self._pipes[k]

    def _generate_local(self, spec: ModelSpec, req: VideoRequest, progress: Optional[Callable[[StepPreview], None]] = None) -> VideoGenerationResult:
        if req.seed is None and self.ranks is not None:
            raise ValueError("a multi-process engine needs VideoRequest.seed (every rank must draw the same noise)")
        pipe = self.pipeline(spec)
        pipe.recipe.check_request(req)
        return pipe.generate(apply_recipe_defaults(spec, req, pipe.recipe), progress or self._progress)


def Vae3dDecoderCfg(tiny: bool, wan_cfg):
    from ..models.vae.vae3d import WAN_VAE
    from .recipes import wan_tiny_vae_config
    return wan_tiny_vae_config(wan_cfg) if tiny else WAN_VAE
