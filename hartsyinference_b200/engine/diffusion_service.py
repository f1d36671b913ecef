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


def apply_recipe_defaults(spec: ModelSpec, req):
    """A catalog model carries its family's request defaults (steps, guidance, size, frames): fields
    the caller left at the request type's own default take the family's value. (The reference keeps
    these in per-family recipe classes: src/HartsyInference.Engine/Recipes/.)"""
    if not spec.catalog:
        return req
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


def _with_loras(get, keys, loras: tuple):
    """Merge LoRA adapters ((path, strength), ...) into the tensors ``get`` returns."""
    if not loras:
        return get
    from ..assets.lora import LoraStack
    from ..assets.safetensors import SafeTensorsFile
    stack = LoraStack()
    for path, strength in loras:
        f = SafeTensorsFile(path)
        stack.add({k: f.get(k) for k in f.keys()}, float(strength))
    merged = stack.wrap(get, keys)
    if stack.unmatched:
        log.warn(f"[LoRA] {len(stack.unmatched)} adapter module(s) match no weight of the base model (first: {stack.unmatched[0]})")
    return merged


def _load_clip_text(d: Path, tok_dir: Path, device):
    """(encoder, tokenizer) from a diffusers ``text_encoder*`` / ``tokenizer*`` pair, or (None, None)."""
    import json as _json
    from ..assets.tokenizer import ClipTokenizer
    from ..models.encoders.clip import ClipTextEncoder, clip_text_from_hf
    if not (d / "config.json").exists() or not ((tok_dir / "vocab.json").exists() or (tok_dir / "tokenizer.json").exists()):
        return None, None
    cfg = clip_text_from_hf(_json.loads((d / "config.json").read_text()))
    return ClipTextEncoder(cfg, device, get=ShardedCheckpoint(d).get), ClipTokenizer.from_dir(tok_dir, cfg.max_len)


def _load_t5(d: Path, tok_dir: Path, device, fp8: bool):
    import json as _json
    from ..assets.tokenizer import UnigramTokenizer
    from ..models.encoders.t5 import T5Config, T5Encoder
    if not (d / "config.json").exists() or not (tok_dir / "tokenizer.json").exists():
        return None, None
    c = _json.loads((d / "config.json").read_text())
    cfg = T5Config(vocab_size=c["vocab_size"], d_model=c["d_model"], d_kv=c["d_kv"], d_ff=c["d_ff"], num_layers=c["num_layers"],
                   num_heads=c["num_heads"], num_buckets=c.get("relative_attention_num_buckets", 32),
                   max_distance=c.get("relative_attention_max_distance", 128), eps=c.get("layer_norm_epsilon", 1e-6),
                   per_layer_bias=c.get("model_type") == "umt5")
    return T5Encoder(cfg, device, fp8=fp8, get=ShardedCheckpoint(d).get), UnigramTokenizer.from_hf_json(tok_dir / "tokenizer.json")


class ImagesService(_PipelineCache):
    COMMAND = "images.generate"

    def _build(self, spec: ModelSpec, loras: tuple = ()):
        from ..models.dit import flux as F
        from ..models.vae.vae2d import FLUX_VAE, Vae2dDecoder, Vae2dEncoder, tiny_vae2d
        from ..pipelines.flux import FluxComponents, FluxPipeline
        name = spec.requested
        fp8 = bool(config.get("fp8_linears")) and self.device.startswith("cuda")
        tp_comm, cfg_comm = self._comms()
        pl = self.options.placement
        te_dev, vae_dev = self._component_device(pl.text_encoder_device), self._component_device(pl.vae_device)
        if name.startswith("synthetic:sd3"):
            from ..models.dit import sd3 as S3
            from ..pipelines.sd3 import SD3_VAE, Sd3Components, Sd3Pipeline
            tiny = name.endswith("-tiny")
            cfg3 = S3.tiny_sd3() if tiny else S3.SD3_MEDIUM
            dt = torch.bfloat16 if self.device.startswith("cuda") else torch.float32
            vae = Vae2dDecoder(tiny_vae2d() if tiny else SD3_VAE, self.device, dt)
            return Sd3Pipeline(Sd3Components(S3.Sd3Transformer(cfg3, self.device, fp8=fp8 and not tiny), vae))
        if name.startswith("synthetic:"):
            tiny = name.endswith("-tiny")
            if "chroma" in name:
                from ..models.dit import chroma as CH
                cfg = CH.tiny_chroma() if tiny else CH.ChromaConfig()
                tr = CH.ChromaTransformer(cfg, self.device, comm=tp_comm, fp8=fp8 and not tiny)
            else:
                cfg = F.tiny_flux() if tiny else F.FLUX_DEV
                tr = F.FluxTransformer(cfg, self.device, comm=tp_comm, fp8=fp8 and not tiny)
            vae = Vae2dDecoder(tiny_vae2d() if tiny else FLUX_VAE, vae_dev,
                               torch.bfloat16 if self.device.startswith("cuda") else torch.float32)
            if tiny:   # the tiny DiT packs 4 latent channels
                assert cfg.in_channels == 16
            enc = Vae2dEncoder(tiny_vae2d() if tiny else FLUX_VAE, vae_dev, vae.dtype)
            return FluxPipeline(FluxComponents(tr, vae, vae_encoder=enc), cfg_comm=cfg_comm)
        path = Path(spec.local_path or name)
        if not path.exists():
            raise UnsupportedModelError(f"{name}: no such checkpoint")
        ck = ShardedCheckpoint(path / "transformer" if (path / "transformer").exists() else path)
        if ck.get("pos_embed.pos_embed") is not None and ck.get("transformer_blocks.0.norm1_context.linear.weight") is not None:
            # an SD3 / SD3.5 MMDiT (diffusers layout)
            import json as _json
            from ..models.dit import sd3 as S3
            from ..pipelines.sd3 import SD3_VAE, Sd3Components, Sd3Pipeline
            tdir = path / "transformer" if (path / "transformer").exists() else path
            cfg3 = S3.sd3_from_hf(_json.loads((tdir / "config.json").read_text())) if (tdir / "config.json").exists() else S3.SD3_MEDIUM
            vae = None
            if "vae" in spec.aux or (path / "vae").exists():
                vae = Vae2dDecoder(SD3_VAE, self.device, get=ShardedCheckpoint(spec.aux.get("vae", path / "vae")).get)
            comp = Sd3Components(S3.Sd3Transformer(cfg3, self.device, fp8=fp8, get=ck.get), vae)
            cl, cl_tok = _load_clip_text(path / "text_encoder", path / "tokenizer", self.device)
            cg, cg_tok = _load_clip_text(path / "text_encoder_2", path / "tokenizer_2", self.device)
            t5, t5_tok = _load_t5(path / "text_encoder_3", path / "tokenizer_3", self.device, fp8)
            if cl is not None and cg is not None and t5 is not None:
                clip_fn = lambda enc, tok: (lambda prompt: enc.encode(torch.tensor(tok.encode(prompt, pad=True)), layer=-2, project=True))
                comp.clip_l, comp.clip_g = clip_fn(cl, cl_tok), clip_fn(cg, cg_tok)
                comp.t5 = lambda prompt: t5.encode(torch.tensor((t5_tok.encode(prompt)[:256] + [0] * 256)[:256]))
            return Sd3Pipeline(comp)
        # adapters are merged in the checkpoint's own layout (their module names follow it)
        get = _with_loras(ck.get, list(ck.keys()), loras)
        from ..assets.converters import flux_original_to_diffusers, is_flux_original
        if is_flux_original(ck.keys()):
            # a Black Forest Labs / ComfyUI layout file: fused qkv and other names
            renamed = flux_original_to_diffusers({k: get(k) for k in ck.keys()})
            get = renamed.get
            log.decision("Load", f"{path.name}: original Flux layout converted to diffusers names")
        if get("distilled_guidance_layer.in_proj.weight") is not None:
            # Chroma: Flux blocks with the modulation table of an approximator network
            import json as _json
            from ..models.dit import chroma as CH
            tdir = path / "transformer" if (path / "transformer").exists() else path
            cc = _json.loads((tdir / "config.json").read_text()) if (tdir / "config.json").exists() else {}
            ccfg = CH.ChromaConfig(num_double_blocks=int(cc.get("num_layers", 19)), num_single_blocks=int(cc.get("num_single_layers", 38)),
                                   approximator_channels=int(cc.get("approximator_num_channels", 64)),
                                   approximator_hidden=int(cc.get("approximator_hidden_dim", 5120)),
                                   approximator_layers=int(cc.get("approximator_layers", 5)))
            tr = CH.ChromaTransformer(ccfg, self.device, comm=tp_comm, fp8=fp8, get=get)
        else:
            import dataclasses
            base = F.FLUX_DEV
            xw = get("x_embedder.weight")
            if xw is not None and xw.shape[1] != base.in_channels:
                # a Fill / Canny / Depth variant: more input channels than predicted ones
                base = dataclasses.replace(base, in_channels=int(xw.shape[1]), out_channels=base.in_channels)
            if get("time_text_embed.guidance_embedder.linear_1.weight") is None:
                base = dataclasses.replace(base, guidance_embed=False)          # schnell-class checkpoints
            tr = F.FluxTransformer(base, self.device, comm=tp_comm, fp8=fp8, get=get)
        vae = enc = None
        if "vae" in spec.aux or (path / "vae").exists():
            vck = ShardedCheckpoint(spec.aux.get("vae", path / "vae"))
            vae = Vae2dDecoder(FLUX_VAE, vae_dev, get=vck.get)
            if vck.get("encoder.conv_in.weight") is not None:
                enc = Vae2dEncoder(FLUX_VAE, vae_dev, get=vck.get)
        cnet = None
        if "controlnet" in spec.aux:
            import json as _json
            from ..models.dit.flux_controlnet import FluxControlNet
            cdir = Path(spec.aux["controlnet"])
            cc = _json.loads((cdir / "config.json").read_text()) if (cdir / "config.json").exists() else {}
            ccfg = F.FluxConfig(num_double_blocks=int(cc.get("num_layers", 5)), num_single_blocks=int(cc.get("num_single_layers", 10)))
            cnet = FluxControlNet(ccfg, self.device, fp8=fp8, get=ShardedCheckpoint(cdir).get)
        comp = FluxComponents(tr, vae, vae_encoder=enc, controlnet=cnet)
        comp.clip, comp.clip_tokenizer = _load_clip_text(path / "text_encoder", path / "tokenizer", te_dev)
        comp.t5, comp.t5_tokenizer = _load_t5(path / "text_encoder_2", path / "tokenizer_2", te_dev, fp8)
        return FluxPipeline(comp, cfg_comm=cfg_comm)

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
        return self.pipeline(spec, loras).generate(apply_recipe_defaults(spec, req), progress or self._progress)


class VideoService(_PipelineCache):
    COMMAND = "video.generate"

    def _build(self, spec: ModelSpec):
        from ..models.dit import wan as W
        from ..models.vae.vae3d import WAN_VAE, Vae3dDecoder
        from ..pipelines.wan import WanComponents, WanPipeline
        name = spec.requested
        fp8 = bool(config.get("fp8_linears")) and self.device.startswith("cuda")
        dt = torch.bfloat16 if self.device.startswith("cuda") else torch.float32
        sp_comm, cfg_comm = self._comms()
        pl = self.options.placement
        te_dev, vae_dev = self._component_device(pl.text_encoder_device), self._component_device(pl.vae_device)
        if name.startswith("synthetic:"):
            tiny = name.endswith("-tiny")
            cfg = W.tiny_wan() if tiny else (W.WAN_1_3B if "1.3b" in name else W.WAN_14B)
            tr = W.WanTransformer(cfg, self.device, sp_comm=sp_comm, fp8=fp8 and not tiny)
            vae = Vae3dDecoder(Vae3dDecoderCfg(tiny, cfg), vae_dev, dt)
            return WanPipeline(WanComponents(tr, vae), cfg_comm=cfg_comm)
        path = Path(spec.local_path or name)
        if not path.exists():
            raise UnsupportedModelError(f"{name}: no such checkpoint")
        # a diffusers-layout directory keeps the transformer, VAE, umT5 encoder and tokenizer in sub-folders
        ck = ShardedCheckpoint(path / "transformer" if (path / "transformer").exists() else path)
        tr = W.WanTransformer(W.WAN_14B, self.device, sp_comm=sp_comm, fp8=fp8, get=ck.get)
        vae = None
        vae_dir = spec.aux.get("vae") or (str(path / "vae") if (path / "vae").exists() else None)
        if vae_dir:
            vae = Vae3dDecoder(WAN_VAE, vae_dev, dt, get=ShardedCheckpoint(vae_dir).get)
        comp = WanComponents(tr, vae)
        te_dir = Path(spec.aux["text_encoder"]) if "text_encoder" in spec.aux else path / "text_encoder"
        tok_dir = te_dir if (te_dir / "tokenizer.json").exists() else path / "tokenizer"
        comp.text_encoder, comp.tokenizer = _load_t5(te_dir, tok_dir, te_dev, fp8)
        return WanPipeline(comp, cfg_comm=cfg_comm)

    def pipeline(self, spec: ModelSpec):
        k = self.key(spec)
        if k not in self._pipes:
            log.info(f"[Video] constructing pipeline for {spec.requested}")
            self._pipes[k] = self._build(spec)
        return self._pipes[k]

    def _generate_local(self, spec: ModelSpec, req: VideoRequest, progress: Optional[Callable[[StepPreview], None]] = None) -> VideoGenerationResult:
        if req.seed is None and self.ranks is not None:
            raise ValueError("a multi-process engine needs VideoRequest.seed (every rank must draw the same noise)")
        return self.pipeline(spec).generate(apply_recipe_defaults(spec, req), progress or self._progress)


def Vae3dDecoderCfg(tiny: bool, wan_cfg):
    from ..models.vae.vae3d import WAN_VAE, Vae3dConfig
    if not tiny:
        return WAN_VAE
    return Vae3dConfig(z_dim=wan_cfg.in_channels, dim=8, dim_mult=(1, 2, 2, 2), num_res_blocks=1,
                       temporal_upsample=(True, True, False))
