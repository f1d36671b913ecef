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


def _count_controlnet(cfg):
    m = U.ControlNet(cfg, "meta", dtype=torch.float32)
    orig = U.sinusoid
    U.sinusoid = lambda v, d: torch.empty(v.shape[0], d, device="meta")
    try:
        kw = {}
        if cfg.addition_embed_dim:
            kw = dict(pooled=torch.empty(1, cfg.addition_embed_dim - 6 * cfg.addition_time_embed_dim, device="meta"),
                      time_ids=torch.empty(1, 6, device="meta"))
        down, mid = m.forward(torch.empty(1, 4, 8, 8, device="meta"), torch.empty(1, device="meta"),
                              torch.empty(1, 7, cfg.cross_attention_dim, device="meta"), torch.empty(1, 3, 64, 64, device="meta"), **kw)
    finally:
        U.sinusoid = orig
    return sum(v.numel() for v in m._w.values()), down, mid, m


def test_controlnet_structure_matches_the_released_models():
    n, down, mid, m = _count_controlnet(U.SD15)
    assert n == 361_279_120                                     # the published SD 1.5 ControlNets
    assert len(down) == 12 and [d.shape[1] for d in down] == [320] * 4 + [640] * 3 + [1280] * 5 and mid.shape[1] == 1280
    assert [d.shape[-1] for d in down] == [8, 8, 8, 4, 4, 4, 2, 2, 2, 1, 1, 1]
    assert "controlnet_cond_embedding.blocks.5.weight" in m._w and m._w["controlnet_cond_embedding.blocks.5.weight"].shape == (256, 96, 3, 3)
    n, down, mid, _ = _count_controlnet(U.SDXL_BASE)
    assert n == 1_251_014_160 and len(down) == 9                # SDXL ControlNets: 1.25 B


def test_controlnet_residuals_enter_the_unet():
    cfg = U.tiny_unet()
    unet, cn = U.UNet2D(cfg, "cpu", seed=0), U.ControlNet(cfg, "cpu", seed=1)
    lat, ctx = torch.randn(2, 4, 8, 8), torch.randn(2, 5, cfg.cross_attention_dim)
    cond = torch.rand(2, 3, 64, 64)
    base = unet.forward(lat, torch.tensor(10.0), ctx)
    down, mid = cn.forward(lat, torch.tensor(10.0), ctx, cond)
    skips = 1 + len(cfg.block_out_channels) * cfg.layers_per_block + len(cfg.block_out_channels) - 1
    assert len(down) == skips and mid.shape[1] == cfg.block_out_channels[-1]
    with_control = unet.forward(lat, torch.tensor(10.0), ctx, down_residuals=down, mid_residual=mid)
    assert not torch.allclose(with_control, base, atol=1e-4)
    # zero projections (a freshly initialised ControlNet) leave the U-Net untouched; the scale is a plain factor
    zeros = [torch.zeros_like(d) for d in down]
    assert torch.allclose(unet.forward(lat, torch.tensor(10.0), ctx, down_residuals=zeros, mid_residual=torch.zeros_like(mid)), base, atol=1e-6)
    half, _ = cn.forward(lat, torch.tensor(10.0), ctx, cond, scale=0.5)
    assert all(torch.allclose(h, d * 0.5, atol=1e-6) for h, d in zip(half, down))
    # the picture matters, and only through the hint stack
    other, _ = cn.forward(lat, torch.tensor(10.0), ctx, 1.0 - cond)
    assert not torch.allclose(other[0], down[0], atol=1e-5)
    with pytest.raises(ValueError):
        unet.forward(lat, torch.tensor(10.0), ctx, down_residuals=down[:-1], mid_residual=mid)


def test_ip_adapter_adds_decoupled_cross_attention():
    cfg = U.tiny_unet()
    unet = U.UNet2D(cfg, "cpu", seed=0)
    paths = unet.cross_attention_paths()
    # adapters count layers down blocks first, then up blocks, then the middle block
    assert paths[0].startswith("down_blocks") and paths[-1].startswith("mid_block") and any(p.startswith("up_blocks") for p in paths)
    assert len(U.UNet2D(U.SD15, "meta").cross_attention_paths()) == 16 and len(U.UNet2D(U.SDXL_BASE, "meta").cross_attention_paths()) == 70
    g = torch.Generator().manual_seed(3)
    d, e, n_tok = cfg.cross_attention_dim, 24, 4
    sd = {"image_proj.proj.weight": torch.randn(n_tok * d, e, generator=g) * 0.2, "image_proj.proj.bias": torch.zeros(n_tok * d),
          "image_proj.norm.weight": torch.ones(d), "image_proj.norm.bias": torch.zeros(d)}
    widths = {}
    lat, ctx = torch.randn(1, 4, 8, 8), torch.randn(1, 5, d)
    base = unet.forward(lat, torch.tensor(10.0), ctx)
    for name, t in unet._w.items():
        if name.endswith("attn2.to_k.weight"):
            widths[name[:-len(".to_k.weight")]] = t.shape[0]
    for i, pth in enumerate(paths):
        sd[f"ip_adapter.{2 * i + 1}.to_k_ip.weight"] = torch.randn(widths[pth], d, generator=g) * 0.2
        sd[f"ip_adapter.{2 * i + 1}.to_v_ip.weight"] = torch.randn(widths[pth], d, generator=g) * 0.2
    project = U.install_ip_adapter(unet, sd.get)
    tokens = project(torch.randn(1, e, generator=g))
    assert tokens.shape == (1, n_tok, d)
    assert torch.allclose(unet.forward(lat, torch.tensor(10.0), ctx), base, atol=1e-6)               # no picture: the plain model
    with_image = unet.forward(lat, torch.tensor(10.0), ctx, image_tokens=tokens)
    assert not torch.allclose(with_image, base, atol=1e-4)
    assert torch.allclose(unet.forward(lat, torch.tensor(10.0), ctx, image_tokens=tokens, image_scale=0.0), base, atol=1e-6)
    # one layer restated: out = attn(q, k, v) + scale * attn(q, k_ip, v_ip), then the output projection
    p = paths[0]
    c = widths[p]
    heads = cfg.num_heads[0]
    x = torch.randn(1, 6, c, generator=g)
    unet._ip["tokens"], unet._ip["scale"] = tokens, 0.7
    got = unet._attention(x, ctx, p, c, heads, d)
    import torch.nn.functional as F
    split = lambda t: t.view(1, -1, heads, c // heads).transpose(1, 2)
    q = split(F.linear(x, unet._w[p + ".to_q.weight"]))
    k, v = split(F.linear(ctx, unet._w[p + ".to_k.weight"])), split(F.linear(ctx, unet._w[p + ".to_v.weight"]))
    ik, iv = split(F.linear(tokens, sd["ip_adapter.1.to_k_ip.weight"])), split(F.linear(tokens, sd["ip_adapter.1.to_v_ip.weight"]))
    o = F.scaled_dot_product_attention(q, k, v) + 0.7 * F.scaled_dot_product_attention(q, ik, iv)
    want = F.linear(o.transpose(1, 2).reshape(1, 6, c), unet._w[p + ".to_out.0.weight"], unet._w[p + ".to_out.0.bias"])
    assert torch.allclose(got, want, atol=1e-5)
    with pytest.raises(KeyError):
        U.install_ip_adapter(U.UNet2D(cfg, "cpu"), {k: v for k, v in sd.items() if not k.startswith("ip_adapter.1.")}.get)


def test_pipeline_takes_control_and_picture_prompts():
    from hartsyinference_b200.engine.requests import ImageRequest
    from hartsyinference_b200.pipelines.sdxl import SdComponents, StableDiffusionPipeline
    cfg = U.tiny_unet()
    unet = U.UNet2D(cfg, "cpu", seed=0)
    pipe = StableDiffusionPipeline(SdComponents(unet=unet))
    req = ImageRequest(prompt="a cat", width=64, height=64, steps=2, cfg_scale=3.0, seed=5)
    plain = pipe.generate(req)
    with pytest.raises(ValueError):
        pipe.generate(ImageRequest(prompt="a cat", width=64, height=64, steps=2, seed=5, control_image=torch.rand(3, 64, 64)))
    pipe.c.controlnet = U.ControlNet(cfg, "cpu", seed=2)
    cond, neg = pipe.encode_prompt("a cat"), pipe.encode_prompt("")
    z0 = pipe.denoise(cond, neg, 64, 64, 2, 3.0, 5)
    z1 = pipe.denoise(cond, neg, 64, 64, 2, 3.0, 5, control=torch.rand(1, 3, 64, 64))
    z2 = pipe.denoise(cond, neg, 64, 64, 2, 3.0, 5, control=torch.rand(1, 3, 64, 64), control_scale=0.0)
    assert not torch.allclose(z1, z0, atol=1e-4) and torch.allclose(z2, z0, atol=1e-5)
    controlled = pipe.generate(ImageRequest(prompt="a cat", width=64, height=64, steps=2, cfg_scale=3.0, seed=5,
                                            control_image=(torch.rand(32, 32, 3) * 255).to(torch.uint8)))
    assert controlled.width == plain.width and controlled.seed == 5
    with pytest.raises(ValueError):
        pipe.denoise(cond, neg, 64, 64, 1, 3.0, 5, image_embeds=torch.randn(1, 8))


def test_recipe_loads_adapters_beside_the_model(tmp_path):
    from hartsyinference_b200.assets.safetensors import save_file
    from hartsyinference_b200.engine import InferenceEngine
    from hartsyinference_b200.engine.requests import ImageRequest, Modality, ModelSpec
    cfg = U.tiny_unet(True)
    hf = {"block_out_channels": [32, 64], "attention_head_dim": [2, 4], "transformer_layers_per_block": [1, 2], "layers_per_block": 1,
          "down_block_types": ["DownBlock2D", "CrossAttnDownBlock2D"], "up_block_types": ["CrossAttnUpBlock2D", "UpBlock2D"],
          "cross_attention_dim": 48, "use_linear_projection": True, "addition_embed_type": "text_time", "norm_num_groups": 8,
          "projection_class_embeddings_input_dim": 72, "addition_time_embed_dim": 8}
    x, ctx = torch.randn(1, 4, 8, 8), torch.randn(1, 77, 48)
    kw = dict(pooled=torch.randn(1, 24), time_ids=torch.tensor([[32.0, 32, 0, 0, 32, 32]]))
    src = U.UNet2D(cfg, "cpu", seed=3)
    src.forward(x, torch.tensor([100.0]), ctx, **kw)
    cn = U.ControlNet(cfg, "cpu", seed=4)
    want_down, want_mid = cn.forward(x, torch.tensor([100.0]), ctx, torch.rand(1, 3, 64, 64, generator=torch.Generator().manual_seed(0)), **kw)
    d = tmp_path / "xl"
    for sub, model in (("unet", src), ("controlnet", cn)):
        (d / sub).mkdir(parents=True)
        (d / sub / "config.json").write_text(json.dumps(hf))
        save_file({k: v.contiguous() for k, v in model._w.items()}, d / sub / "diffusion_pytorch_model.safetensors")
    g = torch.Generator().manual_seed(5)
    ip = {"image_proj.proj.weight": torch.randn(2 * 48, 16, generator=g) * 0.2, "image_proj.proj.bias": torch.zeros(2 * 48),
          "image_proj.norm.weight": torch.ones(48), "image_proj.norm.bias": torch.zeros(48)}
    for i, pth in enumerate(src.cross_attention_paths()):
        c = src._w[pth + ".to_k.weight"].shape[0]
        ip[f"ip_adapter.{2 * i + 1}.to_k_ip.weight"] = torch.randn(c, 48, generator=g) * 0.2
        ip[f"ip_adapter.{2 * i + 1}.to_v_ip.weight"] = torch.randn(c, 48, generator=g) * 0.2
    (d / "ip_adapter").mkdir()
    save_file(ip, d / "ip_adapter" / "ip-adapter.safetensors")
    eng = InferenceEngine("cpu")
    spec = ModelSpec(str(d), Modality.IMAGE, local_path=str(d))
    pipe = eng.images.pipeline(spec)
    assert pipe.c.controlnet is not None and pipe.c.image_projector is not None and pipe.c.image_encoder is None
    down, mid = pipe.c.controlnet.forward(x, torch.tensor([100.0]), ctx, torch.rand(1, 3, 64, 64, generator=torch.Generator().manual_seed(0)), **kw)
    assert torch.allclose(mid, want_mid, atol=1e-5) and all(torch.allclose(a, b, atol=1e-5) for a, b in zip(down, want_down))
    res = eng.images.generate(spec, ImageRequest(prompt="x", width=32, height=32, steps=2, cfg_scale=3.0, seed=1, control_image=torch.rand(3, 32, 32)))
    assert res.width == 32
    cond, neg = pipe.encode_prompt("x"), pipe.encode_prompt("")
    z0 = pipe.denoise(cond, neg, 32, 32, 2, 3.0, 1)
    z1 = pipe.denoise(cond, neg, 32, 32, 2, 3.0, 1, image_embeds=torch.randn(1, 16, generator=g))
    assert not torch.allclose(z0, z1, atol=1e-4)
    with pytest.raises(ValueError):
        eng.images.generate(spec, ImageRequest(prompt="x", width=32, height=32, steps=1, seed=1, image_prompt=torch.rand(3, 32, 32)))
