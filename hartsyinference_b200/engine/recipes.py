"""Per-family construction recipes for the image and video services.

A recipe knows which family it handles (a catalog slug such as ``flux``, ``chroma``, ``sd3``, ``wan``, or
a tensor-name signature of a bare checkpoint), how to build that family's pipeline from a checkpoint
plus side models (text encoders, VAE, ControlNet) on the devices and process groups of the engine's
placement, which composition features the family supports, and the family's recommended request
defaults. The services keep one registry per modality; adding a family = registering a recipe, and
CLI, HTTP and the C ABI can drive it.

Reference: src/HartsyInference.Engine/Recipes/ (IArchitectureRecipe.cs, RecipeRegistry.cs,
RecipeContext.cs, ImageDefaults.cs, ImageFeatures.cs, Image/Flux1Recipe*.cs, Video/).
"""
from __future__ import annotations

import dataclasses
import enum
import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable, Optional

import torch

from .. import log
from ..assets.safetensors import ShardedCheckpoint
from ..exceptions import UnsupportedModelError
from .requests import EngineOptions, ModelSpec


class Features(enum.Flag):
    NONE = 0
    LORA = enum.auto()
    CONTROLNET = enum.auto()
    IMG2IMG = enum.auto()
    INPAINT = enum.auto()
    TRUE_CFG = enum.auto()            # negative prompt with a second forward pass
    CFG_PARALLEL = enum.auto()        # the two guidance branches on two ranks
    TENSOR_PARALLEL = enum.auto()
    SEQUENCE_PARALLEL = enum.auto()
    STEP_CACHE = enum.auto()


@dataclass(frozen=True)
class Defaults:
    """Request fields a family recommends; applied to the fields the caller left at the request type's
    own default (``apply``)."""
    values: dict = field(default_factory=dict)

    def apply(self, req):
        changes = {}
        for f in dataclasses.fields(req):
            if f.name in self.values and getattr(req, f.name) == f.default:
                changes[f.name] = self.values[f.name]
        return dataclasses.replace(req, **changes) if changes else req


@dataclass
class RecipeContext:
    """What a recipe gets to build a pipeline."""
    spec: ModelSpec
    device: str
    options: EngineOptions
    fp8: bool
    inner_comm: Optional[object]          # tensor- / sequence-parallel group of this rank, or None
    cfg_comm: Optional[object]            # two-rank guidance group, or None
    text_encoder_device: str
    vae_device: str
    loras: tuple = ()
    checkpoint: Optional[ShardedCheckpoint] = None
    root: Optional[Path] = None

    @property
    def dtype(self) -> torch.dtype:
        return torch.bfloat16 if self.device.startswith("cuda") else torch.float32

    def transformer_dir(self) -> Path:
        return self.root / "transformer" if (self.root / "transformer").exists() else self.root

    def transformer_config(self) -> dict:
        p = self.transformer_dir() / "config.json"
        return json.loads(p.read_text()) if p.exists() else {}


class Recipe:
    """Base class; subclasses set ``name`` / ``families`` and implement ``construct`` (and ``detect`` when a
    bare checkpoint of the family can be told by its tensor names)."""
    name = ""
    families: tuple = ()
    supports = Features.NONE
    defaults = Defaults()

    def matches(self, family_id: str) -> bool:
        f = (family_id or "").lower()
        return any(f == x or f.startswith(x + "-") or f.startswith(x + ".") for x in self.families)

    def detect(self, ck: ShardedCheckpoint) -> bool:
        return False

    def construct(self, ctx: RecipeContext):
        raise NotImplementedError

    def check_request(self, req) -> None:
        """Reject composition objects this family does not apply, instead of silently ignoring them."""
        need = Features.NONE
        if getattr(req, "loras", None):
            need |= Features.LORA
        if getattr(req, "control_image", None) is not None:
            need |= Features.CONTROLNET
        if getattr(req, "init_image", None) is not None:
            need |= Features.IMG2IMG
        if getattr(req, "mask_image", None) is not None:
            need |= Features.INPAINT
        missing = need & ~self.supports
        if missing:
            raise UnsupportedModelError(f"the {self.name} recipe does not support: {missing}")


class RecipeRegistry:
    def __init__(self, modality: str):
        self.modality = modality
        self._recipes: list[Recipe] = []

    def register(self, recipe: Recipe, first: bool = False) -> Recipe:
        self._recipes.insert(0, recipe) if first else self._recipes.append(recipe)
        return recipe

    def names(self) -> list[str]:
        return [r.name for r in self._recipes]

    def for_family(self, family_id: Optional[str]) -> Optional[Recipe]:
        if not family_id:
            return None
        return next((r for r in self._recipes if r.matches(family_id)), None)

    def resolve(self, spec: ModelSpec, ck: Optional[ShardedCheckpoint]) -> Recipe:
        """Family id first (catalog slug, or the name after ``synthetic:``), then tensor signatures."""
        fam = None
        if spec.requested.startswith("synthetic:"):
            fam = spec.requested[len("synthetic:"):]
        elif spec.catalog:
            from ..assets.catalog import ModelCatalog
            entry = ModelCatalog().find(spec.catalog)
            fam = getattr(entry, "family", None) or spec.catalog
        r = self.for_family(fam)
        if r is None and ck is not None:
            r = next((x for x in self._recipes if x.detect(ck)), None)
        if r is None:
            raise UnsupportedModelError(f"{spec.requested}: no {self.modality} recipe matches (registered: {', '.join(self.names())})")
        log.decision("Load", f"{spec.requested}: {self.modality} recipe '{r.name}'")
        return r


# ------------------------------------------------------------------------------------ shared loaders
def with_loras(get, keys, loras: tuple):
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


def load_clip_text(d: Path, tok_dir: Path, device):
    """(encoder, tokenizer) from a diffusers ``text_encoder*`` / ``tokenizer*`` pair, or (None, None)."""
    import json as _json
    from ..assets.tokenizer import ClipTokenizer
    from ..models.encoders.clip import ClipTextEncoder, clip_text_from_hf
    if not (d / "config.json").exists() or not ((tok_dir / "vocab.json").exists() or (tok_dir / "tokenizer.json").exists()):
        return None, None
    cfg = clip_text_from_hf(_json.loads((d / "config.json").read_text()))
    return ClipTextEncoder(cfg, device, get=ShardedCheckpoint(d).get), ClipTokenizer.from_dir(tok_dir, cfg.max_len)


def load_t5(d: Path, tok_dir: Path, device, fp8: bool):
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



IMAGE_RECIPES = RecipeRegistry("image")
VIDEO_RECIPES = RecipeRegistry("video")


# ------------------------------------------------------------------------------------ image families
def _vae_pair(ctx: RecipeContext, cfg, vae_dir):
    """(decoder, encoder or None) of a 2-D VAE directory on the placement's VAE device."""
    from ..models.vae.vae2d import Vae2dDecoder, Vae2dEncoder
    vck = ShardedCheckpoint(vae_dir)
    dec = Vae2dDecoder(cfg, ctx.vae_device, get=vck.get)
    enc = Vae2dEncoder(cfg, ctx.vae_device, get=vck.get) if vck.get("encoder.conv_in.weight") is not None else None
    return dec, enc


class FluxRecipe(Recipe):
    """Flux.1 dev / schnell / Fill / Canny / Depth (diffusers or original layout), optional ControlNet."""
    name = "flux"
    families = ("flux", "flux1", "flux.1")
    supports = (Features.LORA | Features.CONTROLNET | Features.IMG2IMG | Features.INPAINT | Features.TRUE_CFG |
                Features.CFG_PARALLEL | Features.TENSOR_PARALLEL | Features.STEP_CACHE)
    defaults = Defaults({"steps": 20, "guidance": 3.5, "width": 1024, "height": 1024})

    def detect(self, ck):
        return (ck.get("x_embedder.weight") is not None and ck.get("single_transformer_blocks.0.attn.to_q.weight") is not None) or \
            ck.get("double_blocks.0.img_attn.qkv.weight") is not None

    def _stream(self, ctx, weight_bytes: int) -> bool:
        """Ask the VRAM planner where the denoiser's weights go (tensor-parallel shards stay resident)."""
        from .vram_planner import Placement, VramPlanner, resolve_mode
        planner = VramPlanner(ctx.device, ctx.spec.requested, resolve_mode(ctx.options.low_vram))
        # activations of a 1024 x 1024 step: a few dozen [tokens, 4 x hidden] bf16 buffers
        reserve = 3 << 30
        return planner.plan_phase("denoise", weight_bytes, reserve, can_stream=ctx.inner_comm is None) == Placement.STREAMED

    def _transformer(self, ctx, get):
        from ..models.dit import flux as F
        from .vram_planner import checkpoint_bytes
        base = F.FLUX_DEV
        xw = get("x_embedder.weight")
        if xw is not None and xw.shape[1] != base.in_channels:
            # a Fill / Canny / Depth variant: more input channels than predicted ones
            base = dataclasses.replace(base, in_channels=int(xw.shape[1]), out_channels=base.in_channels)
        if get("time_text_embed.guidance_embedder.linear_1.weight") is None:
            base = dataclasses.replace(base, guidance_embed=False)          # schnell-class checkpoints
        stream = self._stream(ctx, checkpoint_bytes(ctx.checkpoint, ctx.fp8, ctx.inner_comm.world if ctx.inner_comm else 1))
        return F.FluxTransformer(base, ctx.device, comm=ctx.inner_comm, fp8=ctx.fp8, get=get, stream_blocks=stream)

    def construct(self, ctx: RecipeContext):
        from ..assets.converters import flux_original_to_diffusers, is_flux_original
        from ..models.dit import flux as F
        from ..models.vae.vae2d import FLUX_VAE, Vae2dDecoder, Vae2dEncoder, tiny_vae2d
        from ..pipelines.flux import FluxComponents, FluxPipeline
        spec = ctx.spec
        if ctx.checkpoint is None:                          # synthetic:flux-dev[-tiny]
            tiny = spec.requested.endswith("-tiny")
            cfg = F.tiny_flux() if tiny else F.FLUX_DEV
            tr = self._synthetic_transformer(ctx, tiny)
            vae = Vae2dDecoder(tiny_vae2d() if tiny else FLUX_VAE, ctx.vae_device, ctx.dtype)
            enc = Vae2dEncoder(tiny_vae2d() if tiny else FLUX_VAE, ctx.vae_device, vae.dtype)
            return FluxPipeline(FluxComponents(tr, vae, vae_encoder=enc), cfg_comm=ctx.cfg_comm)
        ck, path = ctx.checkpoint, ctx.root
        # adapters are merged in the checkpoint's own layout (their module names follow it)
        get = with_loras(ck.get, list(ck.keys()), ctx.loras)
        if is_flux_original(ck.keys()):
            # a Black Forest Labs / ComfyUI layout file: fused qkv and other names
            renamed = flux_original_to_diffusers({k: get(k) for k in ck.keys()})
            get = renamed.get
            log.decision("Load", f"{path.name}: original Flux layout converted to diffusers names")
        tr = self._transformer(ctx, get)
        vae = enc = None
        if "vae" in spec.aux or (path / "vae").exists():
            vae, enc = _vae_pair(ctx, FLUX_VAE, spec.aux.get("vae", path / "vae"))
        cnet = None
        if "controlnet" in spec.aux:
            from ..models.dit.flux_controlnet import FluxControlNet
            cdir = Path(spec.aux["controlnet"])
            cc = json.loads((cdir / "config.json").read_text()) if (cdir / "config.json").exists() else {}
            ccfg = F.FluxConfig(num_double_blocks=int(cc.get("num_layers", 5)), num_single_blocks=int(cc.get("num_single_layers", 10)))
            cnet = FluxControlNet(ccfg, ctx.device, fp8=ctx.fp8, get=ShardedCheckpoint(cdir).get)
        comp = FluxComponents(tr, vae, vae_encoder=enc, controlnet=cnet)
        comp.clip, comp.clip_tokenizer = load_clip_text(path / "text_encoder", path / "tokenizer", ctx.text_encoder_device)
        comp.t5, comp.t5_tokenizer = load_t5(path / "text_encoder_2", path / "tokenizer_2", ctx.text_encoder_device, ctx.fp8)
        self._redux(comp, path, spec, ctx)
        return FluxPipeline(comp, cfg_comm=ctx.cfg_comm)

    @staticmethod
    def _redux(comp, path: Path, spec, ctx) -> None:
        """Optional picture prompts: ``redux/`` (the projector file) with ``image_encoder/`` (SigLIP vision tower);
        ``spec.aux`` may name them elsewhere (``redux``, ``image_encoder``)."""
        rdir = Path(spec.aux.get("redux", path / "redux"))
        edir = Path(spec.aux.get("image_encoder", path / "image_encoder"))
        if not rdir.exists() or not (edir / "config.json").exists():
            return
        from ..models.dit.redux import ReduxImageEncoder
        from ..models.encoders.clip_vision import CLIP_MEAN, CLIP_STD, preprocess_image
        from ..models.encoders.vit import VitEncoder, vit_from_hf
        rck = ShardedCheckpoint(rdir)
        comp.redux = ReduxImageEncoder(rck.get, ctx.device, ctx.dtype)
        raw = json.loads((edir / "config.json").read_text())
        vit = VitEncoder(vit_from_hf({**raw.get("vision_config", raw), "model_type": "siglip"}), ctx.text_encoder_device,
                         get=ShardedCheckpoint(edir).get)
        cm, cs = torch.tensor(CLIP_MEAN)[:, None, None], torch.tensor(CLIP_STD)[:, None, None]

        def states(picture):
            x = preprocess_image(picture, vit.cfg.image_size) * cs + cm          # back to [0, 1], then SigLIP's 0.5 / 0.5
            return vit.hidden_states((x - 0.5) / 0.5)

        comp.image_states = states

    def _synthetic_transformer(self, ctx, tiny):
        from ..models.dit import flux as F
        from .vram_planner import LowVramMode, resolve_mode
        stream = resolve_mode(ctx.options.low_vram) == LowVramMode.ON and ctx.inner_comm is None and ctx.device.startswith("cuda")
        return F.FluxTransformer(F.tiny_flux() if tiny else F.FLUX_DEV, ctx.device, comm=ctx.inner_comm, fp8=ctx.fp8 and not tiny,
                                 stream_blocks=stream)


class ChromaRecipe(FluxRecipe):
    """Chroma: Flux blocks whose modulation vectors come from an approximator network; true CFG, no
    pooled / guidance conditioning."""
    name = "chroma"
    families = ("chroma", "chroma1")
    supports = FluxRecipe.supports & ~Features.CONTROLNET
    defaults = Defaults({"steps": 30, "cfg_scale": 4.0, "width": 1024, "height": 1024})

    def detect(self, ck):
        return ck.get("distilled_guidance_layer.in_proj.weight") is not None

    def _transformer(self, ctx, get):
        from ..models.dit import chroma as CH
        cc = ctx.transformer_config()
        ccfg = CH.ChromaConfig(num_double_blocks=int(cc.get("num_layers", 19)), num_single_blocks=int(cc.get("num_single_layers", 38)),
                               approximator_channels=int(cc.get("approximator_num_channels", 64)),
                               approximator_hidden=int(cc.get("approximator_hidden_dim", 5120)),
                               approximator_layers=int(cc.get("approximator_layers", 5)))
        return CH.ChromaTransformer(ccfg, ctx.device, comm=ctx.inner_comm, fp8=ctx.fp8, get=get)

    def _synthetic_transformer(self, ctx, tiny):
        from ..models.dit import chroma as CH
        return CH.ChromaTransformer(CH.tiny_chroma() if tiny else CH.ChromaConfig(), ctx.device, comm=ctx.inner_comm,
                                    fp8=ctx.fp8 and not tiny)


class Sd3Recipe(Recipe):
    """Stable Diffusion 3 / 3.5 MMDiT (diffusers layout): CLIP-L + CLIP-G + T5 conditioning, true CFG."""
    name = "sd3"
    families = ("sd3", "sd3.5", "sd35", "stable-diffusion-3")
    supports = Features.TRUE_CFG
    defaults = Defaults({"steps": 28, "cfg_scale": 4.5, "width": 1024, "height": 1024})

    def detect(self, ck):
        return ck.get("pos_embed.pos_embed") is not None and ck.get("transformer_blocks.0.norm1_context.linear.weight") is not None

    def construct(self, ctx: RecipeContext):
        from ..models.dit import sd3 as S3
        from ..models.vae.vae2d import Vae2dDecoder, tiny_vae2d
        from ..pipelines.sd3 import SD3_VAE, Sd3Components, Sd3Pipeline
        spec = ctx.spec
        if ctx.checkpoint is None:
            tiny = spec.requested.endswith("-tiny")
            cfg3 = S3.tiny_sd3() if tiny else S3.SD3_MEDIUM
            vae = Vae2dDecoder(tiny_vae2d() if tiny else SD3_VAE, ctx.device, ctx.dtype)
            return Sd3Pipeline(Sd3Components(S3.Sd3Transformer(cfg3, ctx.device, fp8=ctx.fp8 and not tiny), vae))
        ck, path = ctx.checkpoint, ctx.root
        tc = ctx.transformer_config()
        cfg3 = S3.sd3_from_hf(tc) if tc else S3.SD3_MEDIUM
        vae = None
        if "vae" in spec.aux or (path / "vae").exists():
            vae = Vae2dDecoder(SD3_VAE, ctx.device, get=ShardedCheckpoint(spec.aux.get("vae", path / "vae")).get)
        comp = Sd3Components(S3.Sd3Transformer(cfg3, ctx.device, fp8=ctx.fp8, get=ck.get), vae)
        cl, cl_tok = load_clip_text(path / "text_encoder", path / "tokenizer", ctx.device)
        cg, cg_tok = load_clip_text(path / "text_encoder_2", path / "tokenizer_2", ctx.device)
        t5, t5_tok = load_t5(path / "text_encoder_3", path / "tokenizer_3", ctx.device, ctx.fp8)
        if cl is not None and cg is not None and t5 is not None:
            clip_fn = lambda enc, tok: (lambda prompt: enc.encode(torch.tensor(tok.encode(prompt, pad=True)), layer=-2, project=True))
            comp.clip_l, comp.clip_g = clip_fn(cl, cl_tok), clip_fn(cg, cg_tok)
            comp.t5 = lambda prompt: t5.encode(torch.tensor((t5_tok.encode(prompt)[:256] + [0] * 256)[:256]))
        return Sd3Pipeline(comp)


class StableDiffusionRecipe(Recipe):
    """Stable Diffusion 1.5 and SDXL (diffusers layout: ``unet/``, ``vae/``, ``text_encoder[_2]/``,
    ``tokenizer[_2]/``): convolutional U-Net, CLIP conditioning, epsilon prediction, true CFG."""
    name = "stable-diffusion"
    families = ("sdxl", "sd15", "sd1.5", "sd-1.5", "stable-diffusion-xl", "stable-diffusion-v1", "stable-diffusion-1")
    supports = Features.TRUE_CFG | Features.CONTROLNET
    defaults = Defaults({"steps": 30, "cfg_scale": 7.0, "width": 1024, "height": 1024})

    def detect(self, ck):
        return ck.get("down_blocks.0.resnets.0.conv1.weight") is not None and ck.get("time_embedding.linear_1.weight") is not None

    def construct(self, ctx: RecipeContext):
        from ..models.unet import unet2d as U
        from ..models.vae.vae2d import Vae2dDecoder, tiny_vae2d
        from ..pipelines.sdxl import SD15_VAE, SDXL_VAE, SdComponents, StableDiffusionPipeline
        spec = ctx.spec
        if ctx.checkpoint is None:
            fam = spec.requested[len("synthetic:"):]
            tiny, xl = fam.endswith("-tiny"), fam.startswith("sdxl") or "xl" in fam.split("-")[0]
            cfg = U.tiny_unet(xl) if tiny else (U.SDXL_BASE if xl else U.SD15)
            vae = Vae2dDecoder(tiny_vae2d() if tiny else (SDXL_VAE if xl else SD15_VAE), ctx.device, ctx.dtype)
            return StableDiffusionPipeline(SdComponents(U.UNet2D(cfg, ctx.device), vae))
        path = ctx.root
        udir = path / "unet" if (path / "unet").exists() else path
        ucfg_path = udir / "config.json"
        cfg = U.unet_from_hf(json.loads(ucfg_path.read_text())) if ucfg_path.exists() else U.SD15
        ck = ctx.checkpoint                      # the service opens ``unet/`` when the directory has one
        xl = cfg.addition_embed_dim > 0
        vae = None
        if "vae" in spec.aux or (path / "vae").exists():
            vae = Vae2dDecoder(SDXL_VAE if xl else SD15_VAE, ctx.vae_device, get=ShardedCheckpoint(spec.aux.get("vae", path / "vae")).get)
        comp = SdComponents(U.UNet2D(cfg, ctx.device, get=ck.get), vae)
        cl, cl_tok = load_clip_text(path / "text_encoder", path / "tokenizer", ctx.text_encoder_device)
        if cl is not None:
            layer = -2 if xl else -1
            comp.clip_l = lambda prompt: cl.encode(torch.tensor(cl_tok.encode(prompt, pad=True)), layer=layer)
        if xl:
            cg, cg_tok = load_clip_text(path / "text_encoder_2", path / "tokenizer_2", ctx.text_encoder_device)
            if cg is not None:
                comp.clip_g = lambda prompt: cg.encode(torch.tensor(cg_tok.encode(prompt, pad=True)), layer=-2, project=True)
        self._adapters(comp, cfg, path, spec, ctx)
        return StableDiffusionPipeline(comp)

    @staticmethod
    def _adapters(comp, cfg, path: Path, spec, ctx) -> None:
        """Optional adapters beside the model: ``controlnet/`` (diffusers ControlNet of the same family),
        ``ip_adapter/`` (one adapter file) with ``image_encoder/`` (CLIP vision tower with projection). ``spec.aux``
        may name them elsewhere (``controlnet``, ``ip_adapter``, ``image_encoder``)."""
        from ..models.unet import unet2d as U
        cdir = Path(spec.aux.get("controlnet", path / "controlnet"))
        if cdir.is_dir() and ((cdir / "config.json").exists() or any(cdir.glob("*.safetensors"))):
            ccfg = U.unet_from_hf(json.loads((cdir / "config.json").read_text())) if (cdir / "config.json").exists() else cfg
            comp.controlnet = U.ControlNet(ccfg, ctx.device, get=ShardedCheckpoint(cdir).get)
        adir = Path(spec.aux.get("ip_adapter", path / "ip_adapter"))
        if adir.exists():
            from ..assets.safetensors import SafeTensorsFile
            files = [adir] if adir.is_file() else sorted(adir.glob("*.safetensors"))
            if files:
                f = SafeTensorsFile(files[0])
                names = set(f.keys())
                comp.image_projector = U.install_ip_adapter(comp.unet, lambda n: f.get(n) if n in names else None)
        edir = Path(spec.aux.get("image_encoder", path / "image_encoder"))
        if comp.image_projector is not None and (edir / "config.json").exists():
            from ..models.encoders.clip_vision import ClipVisionEncoder, clip_vision_from_hf, preprocess_image
            raw = json.loads((edir / "config.json").read_text())
            eck = ShardedCheckpoint(edir)
            vision = ClipVisionEncoder(clip_vision_from_hf(raw.get("vision_config", raw)), ctx.text_encoder_device, get=eck.get,
                                       prefix="vision_model.")
            proj = eck.get("visual_projection.weight").float().to(vision.device)
            comp.image_encoder = lambda picture: (vision.embed(preprocess_image(picture, vision.cfg.image_size)).float() @ proj.t())[None]


# ------------------------------------------------------------------------------------ video families
def wan_tiny_vae_config(wan_cfg):
    from ..models.vae.vae3d import Vae3dConfig
    return Vae3dConfig(z_dim=wan_cfg.in_channels, dim=8, dim_mult=(1, 2, 2, 2), num_res_blocks=1,
                       temporal_upsample=(True, True, False))


class WanRecipe(Recipe):
    """Wan 2.1 text-to-video (14B / 1.3B): umT5 encoder, causal 3-D VAE, sequence-parallel transformer."""
    name = "wan"
    families = ("wan", "wan2.1", "wan2")
    supports = Features.TRUE_CFG | Features.CFG_PARALLEL | Features.SEQUENCE_PARALLEL
    defaults = Defaults({"steps": 50, "cfg_scale": 5.0, "width": 832, "height": 480, "frames": 81})

    def detect(self, ck):
        return ck.get("blocks.0.self_attn.q.weight") is not None or ck.get("blocks.0.attn1.to_q.weight") is not None

    def construct(self, ctx: RecipeContext):
        from ..models.dit import wan as W
        from ..models.vae.vae3d import WAN_VAE, Vae3dDecoder
        from ..pipelines.wan import WanComponents, WanPipeline
        spec = ctx.spec
        if ctx.checkpoint is None:
            tiny = spec.requested.endswith("-tiny")
            cfg = W.tiny_wan() if tiny else (W.WAN_1_3B if "1.3b" in spec.requested else W.WAN_14B)
            tr = W.WanTransformer(cfg, ctx.device, sp_comm=ctx.inner_comm, fp8=ctx.fp8 and not tiny)
            vae = Vae3dDecoder(wan_tiny_vae_config(cfg) if tiny else WAN_VAE, ctx.vae_device, ctx.dtype)
            return WanPipeline(WanComponents(tr, vae), cfg_comm=ctx.cfg_comm)
        ck, path = ctx.checkpoint, ctx.root
        tr = W.WanTransformer(W.WAN_14B, ctx.device, sp_comm=ctx.inner_comm, fp8=ctx.fp8, get=ck.get)
        vae = None
        vae_dir = spec.aux.get("vae") or (str(path / "vae") if (path / "vae").exists() else None)
        if vae_dir:
            vae = Vae3dDecoder(WAN_VAE, ctx.vae_device, ctx.dtype, get=ShardedCheckpoint(vae_dir).get)
        comp = WanComponents(tr, vae)
        te_dir = Path(spec.aux["text_encoder"]) if "text_encoder" in spec.aux else path / "text_encoder"
        tok_dir = te_dir if (te_dir / "tokenizer.json").exists() else path / "tokenizer"
        comp.text_encoder, comp.tokenizer = load_t5(te_dir, tok_dir, ctx.text_encoder_device, ctx.fp8)
        return WanPipeline(comp, cfg_comm=ctx.cfg_comm)


# detection order matters where signatures nest: Chroma carries Flux's tensors plus its approximator
IMAGE_RECIPES.register(ChromaRecipe())
IMAGE_RECIPES.register(Sd3Recipe())
IMAGE_RECIPES.register(FluxRecipe())
IMAGE_RECIPES.register(StableDiffusionRecipe())
VIDEO_RECIPES.register(WanRecipe())
