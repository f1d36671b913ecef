"""Stable Diffusion 1.5 / SDXL U-Net (models/unet/unet2d.py), pipeline and recipe. No diffusers package
is available offline, so the structure is pinned by the published parameter counts of the released
checkpoints (every tensor name and shape the forward pass asks for, traced on the meta device) and by
behavioural checks on a tiny random model."""
import json

import pytest
import torch

from hartsyinference_b200.models.unet import unet2d as U


def _trace(cfg, pooled_dim=0, ids=6):
    u = U.UNet2D(cfg, "meta", dtype=torch.float32)
    seen = {}

    def tensor(name, shape, kind="weight"):
        seen[name] = tuple(shape)
        return torch.empty(shape, device="meta")

    u._tensor = tensor
    orig = U.sinusoid
    U.sinusoid = lambda v, d: torch.empty(v.shape[0], d, device="meta")
    try:
        kw = dict(pooled=torch.empty(1, pooled_dim, device="meta"), time_ids=torch.empty(1, ids, device="meta")) if pooled_dim else {}
        y = u.forward(torch.empty(1, 4, 64, 64, device="meta"), torch.empty(1, device="meta"),
                      torch.empty(1, 77, cfg.cross_attention_dim, device="meta"), **kw)
    finally:
        U.sinusoid = orig
    assert y.shape == (1, 4, 64, 64)
    n = 0
    for s in seen.values():
        k = 1
        for v in s:
            k *= v
        n += k
    return seen, n


def test_parameter_counts_of_the_released_models():
    sd15, n15 = _trace(U.SD15)
    assert len(sd15) == 686 and n15 == 859_520_964
    xl, nxl = _trace(U.SDXL_BASE, 1280)
    assert len(xl) == 1680 and nxl == 2_567_463_684
    # a few names and shapes of the diffusers layout
    assert sd15["down_blocks.0.attentions.1.transformer_blocks.0.attn2.to_k.weight"] == (320, 768)
    assert sd15["down_blocks.0.attentions.0.proj_in.weight"] == (320, 320, 1, 1)
    assert sd15["up_blocks.1.resnets.0.conv1.weight"] == (1280, 2560, 3, 3) and "up_blocks.0.attentions.0.norm.weight" not in sd15
    assert xl["down_blocks.2.attentions.1.transformer_blocks.9.ff.net.0.proj.weight"] == (10240, 1280)
    assert xl["add_embedding.linear_1.weight"] == (1280, 2816) and xl["mid_block.attentions.0.proj_in.weight"] == (1280, 1280)
    assert xl["up_blocks.0.resnets.2.conv_shortcut.weight"] == (1280, 1920, 1, 1) and "down_blocks.0.attentions.0.norm.weight" not in xl
    ref, _ = _trace(U.SDXL_REFINER, 1280, ids=5)
    assert ref["add_embedding.linear_1.weight"] == (1536, 2560)


def test_config_from_diffusers_json():
    d = {"block_out_channels": [320, 640, 1280], "attention_head_dim": [5, 10, 20], "transformer_layers_per_block": [1, 2, 10],
         "down_block_types": ["DownBlock2D", "CrossAttnDownBlock2D", "CrossAttnDownBlock2D"],
         "up_block_types": ["CrossAttnUpBlock2D", "CrossAttnUpBlock2D", "UpBlock2D"], "cross_attention_dim": 2048,
         "use_linear_projection": True, "addition_embed_type": "text_time", "projection_class_embeddings_input_dim": 2816,
         "addition_time_embed_dim": 256}
    assert U.unet_from_hf(d) == U.SDXL_BASE
    assert U.unet_from_hf({"attention_head_dim": 8}) == U.SD15


@pytest.mark.parametrize("sdxl", [False, True])
def test_tiny_model_behaviour(sdxl):
    cfg = U.tiny_unet(sdxl)
    u = U.UNet2D(cfg, "cpu", seed=1)
    torch.manual_seed(0)
    x, ctx = torch.randn(2, 4, 16, 16), torch.randn(2, 7, 48)
    kw = dict(pooled=torch.randn(2, 24), time_ids=torch.tensor([[64.0, 64, 0, 0, 64, 64]] * 2)) if sdxl else {}
    t = torch.tensor([500.0, 20.0])
    y = u.forward(x, t, ctx, **kw)
    assert y.shape == x.shape and torch.isfinite(y).all()
    # samples of a batch do not mix; text, timestep (and SDXL's extra conditioning) all reach the output
    x2 = x.clone(); x2[1] += 1
    assert torch.allclose(u.forward(x2, t, ctx, **kw)[0], y[0], atol=1e-5)
    ctx2 = ctx.clone(); ctx2[0] += 1
    assert not torch.allclose(u.forward(x, t, ctx2, **kw)[0], y[0], atol=1e-4)
    assert not torch.allclose(u.forward(x, torch.tensor([900.0, 20.0]), ctx, **kw)[0], y[0], atol=1e-4)
    if sdxl:
        kw2 = dict(kw, time_ids=torch.tensor([[128.0, 64, 0, 0, 64, 64]] * 2))
        assert not torch.allclose(u.forward(x, t, ctx, **kw2), y, atol=1e-5)
        with pytest.raises(ValueError):
            u.forward(x, t, ctx)
    e = U.sinusoid(torch.tensor([3.0]), 8)
    assert torch.allclose(e[0, :4], torch.cos(3.0 * torch.exp(-torch.log(torch.tensor(10000.0)) * torch.arange(4) / 4)))


def test_pipeline_and_recipe_through_the_image_service():
    from hartsyinference_b200.engine import InferenceEngine
    from hartsyinference_b200.engine.requests import ImageRequest, Modality, ModelSpec
    eng = InferenceEngine("cpu")
    for name in ("synthetic:sdxl-tiny", "synthetic:sd15-tiny"):
        req = ImageRequest(prompt="a red cube", negative_prompt="blurry", width=32, height=32, steps=3, cfg_scale=5.0, seed=7)
        a = eng.images.generate(ModelSpec(name, Modality.IMAGE), req)
        b = eng.images.generate(ModelSpec(name, Modality.IMAGE), req)
        assert a.width == 32 and a.height == 32 and a.rgb == b.rgb and a.meta["scheduler"] == "euler_discrete"
        c = eng.images.generate(ModelSpec(name, Modality.IMAGE), ImageRequest(prompt="a blue ball", width=32, height=32, steps=3,
                                                                            cfg_scale=5.0, seed=7))
        assert c.rgb != a.rgb


def test_recipe_loads_a_diffusers_layout_directory(tmp_path):
    from hartsyinference_b200.assets.safetensors import save_file
    from hartsyinference_b200.engine import InferenceEngine
    from hartsyinference_b200.engine.requests import ImageRequest, Modality, ModelSpec
    cfg = U.tiny_unet(True)
    src = U.UNet2D(cfg, "cpu", seed=3)
    x, ctx = torch.randn(1, 4, 8, 8), torch.randn(1, 77, 48)
    kw = dict(pooled=torch.randn(1, 24), time_ids=torch.tensor([[32.0, 32, 0, 0, 32, 32]]))
    want = src.forward(x, torch.tensor([100.0]), ctx, **kw)           # touches (and so creates) every tensor
    d = tmp_path / "xl"
    (d / "unet").mkdir(parents=True)
    (d / "unet" / "config.json").write_text(json.dumps({
        "block_out_channels": [32, 64], "attention_head_dim": [2, 4], "transformer_layers_per_block": [1, 2], "layers_per_block": 1,
        "down_block_types": ["DownBlock2D", "CrossAttnDownBlock2D"], "up_block_types": ["CrossAttnUpBlock2D", "UpBlock2D"],
        "cross_attention_dim": 48, "use_linear_projection": True, "addition_embed_type": "text_time", "norm_num_groups": 8,
        "projection_class_embeddings_input_dim": 72, "addition_time_embed_dim": 8}))
    save_file({k: v.contiguous() for k, v in src._w.items()}, d / "unet" / "diffusion_pytorch_model.safetensors")
    eng = InferenceEngine("cpu")
    spec = ModelSpec(str(d), Modality.IMAGE, local_path=str(d))
    res = eng.images.generate(spec, ImageRequest(prompt="x", width=32, height=32, steps=2, cfg_scale=3.0, seed=1))
    assert res.width == 32
    pipe = eng.images.pipeline(spec)
    assert pipe.sdxl and pipe.c.unet.cfg == cfg
    got = pipe.c.unet.forward(x, torch.tensor([100.0]), ctx, **kw)
    assert torch.allclose(got, want, atol=1e-5)
