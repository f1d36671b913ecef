"""SD3 MMDiT against an independent fp32 statement of the same network, and the pipeline."""
import math

import pytest
import torch
import torch.nn.functional as F

from hartsyinference_b200.models.dit.sd3 import Sd3Transformer, sd3_from_hf, sincos_2d, tiny_sd3


def _weights(cfg, seed=0):
    g = torch.Generator().manual_seed(seed)
    H, D, C, P = cfg.hidden_size, cfg.head_dim, cfg.in_channels, cfg.patch
    w = {}

    def lin(n, o, i, s=1.0):
        w[n + ".weight"] = (torch.randn(o, i, generator=g) * s / math.sqrt(i)).to(torch.bfloat16).float()
        w[n + ".bias"] = (torch.randn(o, generator=g) * 0.05).to(torch.bfloat16).float()
    w["pos_embed.proj.weight"] = (torch.randn(H, C, P, P, generator=g) / math.sqrt(C * P * P)).to(torch.bfloat16).float()
    w["pos_embed.proj.bias"] = torch.zeros(H)
    w["pos_embed.pos_embed"] = sincos_2d(H, cfg.pos_embed_max_size)[None]
    lin("context_embedder", H, cfg.context_dim)
    lin("time_text_embed.timestep_embedder.linear_1", H, 256); lin("time_text_embed.timestep_embedder.linear_2", H, H)
    lin("time_text_embed.text_embedder.linear_1", H, cfg.pooled_dim); lin("time_text_embed.text_embedder.linear_2", H, H)
    for i in range(cfg.num_layers):
        p = f"transformer_blocks.{i}."
        last = i == cfg.num_layers - 1
        lin(p + "norm1.linear", 6 * H, H, 0.5); lin(p + "norm1_context.linear", (2 if last else 6) * H, H, 0.5)
        for n in ("attn.to_q", "attn.to_k", "attn.to_v", "attn.add_q_proj", "attn.add_k_proj", "attn.add_v_proj", "attn.to_out.0"):
            lin(p + n, H, H)
        lin(p + "ff.net.0.proj", cfg.mlp_dim, H); lin(p + "ff.net.2", H, cfg.mlp_dim)
        if not last:
            lin(p + "attn.to_add_out", H, H)
            lin(p + "ff_context.net.0.proj", cfg.mlp_dim, H); lin(p + "ff_context.net.2", H, cfg.mlp_dim)
        if cfg.qk_norm:
            for n in ("attn.norm_q", "attn.norm_k", "attn.norm_added_q", "attn.norm_added_k"):
                w[p + n + ".weight"] = (1 + torch.randn(D, generator=g) * 0.1).to(torch.bfloat16).float()
    lin("norm_out.linear", 2 * H, H, 0.5); lin("proj_out", P * P * C, H)
    return w


def _reference(cfg, w, lat, txt, sigma, pooled):
    """The network written the way the published module computes it, in fp32."""
    H, D, C, P, nh = cfg.hidden_size, cfg.head_dim, cfg.in_channels, cfg.patch, cfg.num_heads
    L = lambda x, n: F.linear(x, w[n + ".weight"], w[n + ".bias"])
    x = F.conv2d(lat, w["pos_embed.proj.weight"], w["pos_embed.proj.bias"], stride=P)        # [1, H, gh, gw]
    gh, gw = x.shape[2:]
    x = x.flatten(2).transpose(1, 2)[0]
    n = cfg.pos_embed_max_size
    pos = w["pos_embed.pos_embed"].reshape(n, n, H)[(n - gh) // 2:(n - gh) // 2 + gh, (n - gw) // 2:(n - gw) // 2 + gw].reshape(-1, H)
    x = x + pos
    c = L(txt[0], "context_embedder")
    half = 128
    freqs = torch.exp(-math.log(10000.0) * torch.arange(half) / half)
    ang = (sigma * 1000.0)[:, None] * freqs[None]
    te = torch.cat([ang.cos(), ang.sin()], -1)
    temb = L(F.silu(L(te, "time_text_embed.timestep_embedder.linear_1")), "time_text_embed.timestep_embedder.linear_2")
    temb = temb + L(F.silu(L(pooled, "time_text_embed.text_embedder.linear_1")), "time_text_embed.text_embedder.linear_2")
    e = F.silu(temb)
    ln = lambda t: F.layer_norm(t, (H,), eps=1e-6)
    rms = lambda t, wt: t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + 1e-6) * wt

    def heads(t, p, names, norms):
        out = []
        for nm, nr in zip(names, norms):
            y = L(t, p + nm).reshape(-1, nh, D)
            if nr is not None and cfg.qk_norm:
                y = rms(y, w[p + nr + ".weight"])
            out.append(y.transpose(0, 1))
        return out

    for i in range(cfg.num_layers):
        p = f"transformer_blocks.{i}."
        last = i == cfg.num_layers - 1
        sh, sc, g1, sh2, sc2, g2 = L(e, p + "norm1.linear")[0].chunk(6)
        xn = ln(x) * (1 + sc) + sh
        if last:
            csc, csh = L(e, p + "norm1_context.linear")[0].chunk(2)
            cn = ln(c) * (1 + csc) + csh
        else:
            csh, csc, cg1, csh2, csc2, cg2 = L(e, p + "norm1_context.linear")[0].chunk(6)
            cn = ln(c) * (1 + csc) + csh
        q, k, v = heads(xn, p, ("attn.to_q", "attn.to_k", "attn.to_v"), ("attn.norm_q", "attn.norm_k", None))
        cq, ck, cv = heads(cn, p, ("attn.add_q_proj", "attn.add_k_proj", "attn.add_v_proj"), ("attn.norm_added_q", "attn.norm_added_k", None))
        a = F.scaled_dot_product_attention(torch.cat([q, cq], 1), torch.cat([k, ck], 1), torch.cat([v, cv], 1))
        a = a.transpose(0, 1).reshape(-1, H)
        S = x.shape[0]
        x = x + g1 * L(a[:S], p + "attn.to_out.0")
        x = x + g2 * L(F.gelu(L(ln(x) * (1 + sc2) + sh2, p + "ff.net.0.proj"), approximate="tanh"), p + "ff.net.2")
        if not last:
            c = c + cg1 * L(a[S:], p + "attn.to_add_out")
            c = c + cg2 * L(F.gelu(L(ln(c) * (1 + csc2) + csh2, p + "ff_context.net.0.proj"), approximate="tanh"), p + "ff_context.net.2")
    sc, sh = L(e, "norm_out.linear")[0].chunk(2)
    out = L(ln(x) * (1 + sc) + sh, "proj_out")
    out = out.reshape(1, gh, gw, P, P, C)
    return torch.einsum("nhwpqc->nchpwq", out).reshape(1, C, gh * P, gw * P)


@pytest.mark.parametrize("qk_norm", [False, True])
def test_sd3_transformer_matches_reference(qk_norm):
    cfg = tiny_sd3(qk_norm=qk_norm)
    w = _weights(cfg)
    m = Sd3Transformer(cfg, "cpu", get=lambda n: w.get(n))
    g = torch.Generator().manual_seed(1)
    lat = torch.randn(1, cfg.in_channels, 8, 12, generator=g)
    txt = torch.randn(1, 7, cfg.context_dim, generator=g)
    pooled = torch.randn(1, cfg.pooled_dim, generator=g)
    sigma = torch.tensor([0.6])
    ref = _reference(cfg, w, lat, txt, sigma, pooled)
    got = m.forward(lat, txt, sigma, pooled).float()
    assert got.shape == ref.shape == lat.shape
    assert torch.nn.functional.cosine_similarity(got.flatten(), ref.flatten(), dim=0) > 0.995
    d = dict(num_layers=3, num_attention_heads=2, attention_head_dim=64, joint_attention_dim=64, pooled_projection_dim=32,
             in_channels=4, pos_embed_max_size=12, qk_norm="rms_norm" if qk_norm else None)
    assert sd3_from_hf(d) == cfg


def test_sd3_pipeline_and_service(tmp_path):
    import json
    from hartsyinference_b200.assets.safetensors import save_file
    from hartsyinference_b200.engine import InferenceEngine, ModelSpec
    from hartsyinference_b200.engine.requests import ImageRequest
    from hartsyinference_b200.pipelines.sd3 import join_conditioning
    eng = InferenceEngine("cpu")
    req = ImageRequest(prompt="a lighthouse", negative_prompt="blurry", width=64, height=64, steps=3, guidance=4.0, seed=5)
    a = eng.images.generate(ModelSpec("synthetic:sd3-tiny"), req)
    b = eng.images.generate(ModelSpec("synthetic:sd3-tiny"), req)
    assert (a.width, a.height) == (64, 64) and a.rgb == b.rgb and a.meta["cfg_scale"] == 4.0 and a.meta["shift"] == 3.0
    c = eng.images.generate(ModelSpec("synthetic:sd3-tiny"), ImageRequest(prompt="a lighthouse", width=64, height=64, steps=3, guidance=1.0, seed=5))
    assert c.rgb != a.rgb                       # without guidance the unconditional pass is skipped

    ctx, pooled = join_conditioning((torch.ones(77, 8), torch.ones(4)), (torch.ones(77, 12), 2 * torch.ones(6)), torch.zeros(5, 32), 32)
    assert ctx.shape == (82, 32) and ctx[0, :20].eq(1).all() and ctx[0, 20:].eq(0).all() and pooled.tolist() == [1] * 4 + [2] * 6

    # a checkpoint directory in the diffusers layout is recognised by its tensors
    cfg = tiny_sd3()
    w = _weights(cfg)
    d = tmp_path / "sd3" / "transformer"
    d.mkdir(parents=True)
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in w.items()}, d / "diffusion_pytorch_model.safetensors")
    (d / "config.json").write_text(json.dumps(dict(num_layers=3, num_attention_heads=2, attention_head_dim=64, joint_attention_dim=64,
                                                   pooled_projection_dim=32, in_channels=4, pos_embed_max_size=12)))
    res = eng.images.generate(ModelSpec(str(tmp_path / "sd3")), ImageRequest(prompt="x", width=32, height=32, steps=2, guidance=2.0, seed=1))
    assert (res.width, res.height) == (32, 32)       # no VAE beside it: a blank canvas of the requested size
    eng.close()
