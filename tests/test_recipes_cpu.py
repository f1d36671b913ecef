"""Recipe registry of the image / video services: family resolution (catalog slug, ``synthetic:`` name,
tensor signature), per-family defaults, rejection of composition features a family does not apply,
and registration of a new family."""
import pytest
import torch

from hartsyinference_b200.engine import recipes as R
from hartsyinference_b200.engine.requests import ImageRequest, ModelSpec, Modality, VideoRequest
from hartsyinference_b200.exceptions import UnsupportedModelError


class _Ck:
    def __init__(self, names):
        self.names = set(names)

    def get(self, k):
        return torch.zeros(1) if k in self.names else None

    def keys(self):
        return list(self.names)


def test_resolution_by_name_and_signature():
    assert R.IMAGE_RECIPES.resolve(ModelSpec("synthetic:flux-dev-tiny", Modality.IMAGE), None).name == "flux"
    assert R.IMAGE_RECIPES.resolve(ModelSpec("synthetic:chroma-tiny", Modality.IMAGE), None).name == "chroma"
    assert R.IMAGE_RECIPES.resolve(ModelSpec("synthetic:sd3-tiny", Modality.IMAGE), None).name == "sd3"
    assert R.VIDEO_RECIPES.resolve(ModelSpec("synthetic:wan-14b", Modality.VIDEO), None).name == "wan"
    flux = _Ck(["x_embedder.weight", "single_transformer_blocks.0.attn.to_q.weight"])
    chroma = _Ck(flux.names | {"distilled_guidance_layer.in_proj.weight"})
    sd3 = _Ck(["pos_embed.pos_embed", "transformer_blocks.0.norm1_context.linear.weight"])
    orig = _Ck(["double_blocks.0.img_attn.qkv.weight"])
    spec = ModelSpec("/some/file", Modality.IMAGE)
    assert R.IMAGE_RECIPES.resolve(spec, flux).name == "flux"
    assert R.IMAGE_RECIPES.resolve(spec, chroma).name == "chroma"        # carries Flux's tensors too: tried first
    assert R.IMAGE_RECIPES.resolve(spec, sd3).name == "sd3"
    assert R.IMAGE_RECIPES.resolve(spec, orig).name == "flux"
    with pytest.raises(UnsupportedModelError):
        R.IMAGE_RECIPES.resolve(spec, _Ck(["something.else"]))


def test_defaults_fill_only_untouched_fields():
    d = R.FluxRecipe().defaults
    req = d.apply(ImageRequest(prompt="x", steps=7))
    assert req.steps == 7 and req.guidance == 3.5
    v = R.WanRecipe().defaults.apply(VideoRequest(prompt="x"))
    assert v.steps == 50 and v.frames == 81 and v.cfg_scale == 5.0


def test_unsupported_features_are_rejected():
    sd3 = R.Sd3Recipe()
    with pytest.raises(UnsupportedModelError):
        sd3.check_request(ImageRequest(prompt="x", loras=[("a.safetensors", 1.0)]))
    R.FluxRecipe().check_request(ImageRequest(prompt="x", loras=[("a.safetensors", 1.0)]))
    with pytest.raises(UnsupportedModelError):
        R.ChromaRecipe().check_request(ImageRequest(prompt="x", control_image=torch.zeros(3, 8, 8)))


def test_registering_a_family():
    reg = R.RecipeRegistry("image")

    class Mine(R.Recipe):
        name = "mine"
        families = ("mine",)
        supports = R.Features.LORA

        def construct(self, ctx):
            return ("pipeline-of", ctx.spec.requested)

    reg.register(Mine())
    r = reg.resolve(ModelSpec("synthetic:mine-v2", Modality.IMAGE), None)
    assert r.name == "mine" and reg.names() == ["mine"]


def test_service_builds_through_the_registry():
    from hartsyinference_b200.engine.inference_engine import InferenceEngine
    eng = InferenceEngine("cpu")
    res = eng.images.generate(ModelSpec("synthetic:flux-dev-tiny", Modality.IMAGE),
                              ImageRequest(prompt="a", width=64, height=64, steps=2, seed=1))
    assert res.width == 64 and len(res.rgb) == 64 * 64 * 3
    pipe = next(iter(eng.images._pipes.values()))
    assert pipe.recipe.name == "flux"
