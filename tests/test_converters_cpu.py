"""Flux checkpoint layouts: original <-> diffusers names, and loading an original-layout file."""
import torch

from hartsyinference_b200.assets.converters import (flux_diffusers_to_original, flux_original_to_diffusers,
                                                    is_flux_original)
from hartsyinference_b200.models.dit import flux as F


def _diffusers_state(cfg, seed=0):
    """Every tensor name the transformer asks for, with random values."""
    g = torch.Generator().manual_seed(seed)
    made = {}
    H, D = cfg.hidden_size, cfg.head_dim
    def lin(n, o, i):
        made[n + ".weight"] = torch.randn(o, i, generator=g) * 0.05
        made[n + ".bias"] = torch.randn(o, generator=g) * 0.05
    lin("x_embedder", H, cfg.in_channels); lin("context_embedder", H, cfg.context_dim)
    lin("time_text_embed.timestep_embedder.linear_1", H, 256); lin("time_text_embed.timestep_embedder.linear_2", H, H)
    lin("time_text_embed.text_embedder.linear_1", H, cfg.pooled_dim); lin("time_text_embed.text_embedder.linear_2", H, H)
    if cfg.guidance_embed:
        lin("time_text_embed.guidance_embedder.linear_1", H, 256); lin("time_text_embed.guidance_embedder.linear_2", H, H)
    for i in range(cfg.num_double_blocks):
        p = f"transformer_blocks.{i}."
        lin(p + "norm1.linear", 6 * H, H); lin(p + "norm1_context.linear", 6 * H, H)
        for n in ("attn.to_q", "attn.to_k", "attn.to_v", "attn.add_q_proj", "attn.add_k_proj", "attn.add_v_proj",
                  "attn.to_out.0", "attn.to_add_out"):
            lin(p + n, H, H)
        for n in ("attn.norm_q", "attn.norm_k", "attn.norm_added_q", "attn.norm_added_k"):
            made[p + n + ".weight"] = 1 + torch.randn(D, generator=g) * 0.1
        lin(p + "ff.net.0.proj", cfg.mlp_dim, H); lin(p + "ff.net.2", H, cfg.mlp_dim)
        lin(p + "ff_context.net.0.proj", cfg.mlp_dim, H); lin(p + "ff_context.net.2", H, cfg.mlp_dim)
    for i in range(cfg.num_single_blocks):
        p = f"single_transformer_blocks.{i}."
        lin(p + "norm.linear", 3 * H, H)
        for n in ("attn.to_q", "attn.to_k", "attn.to_v"):
            lin(p + n, H, H)
        lin(p + "proj_mlp", cfg.mlp_dim, H); lin(p + "proj_out", H, H + cfg.mlp_dim)
        made[p + "attn.norm_q.weight"] = 1 + torch.randn(D, generator=g) * 0.1
        made[p + "attn.norm_k.weight"] = 1 + torch.randn(D, generator=g) * 0.1
    lin("norm_out.linear", 2 * H, H); lin("proj_out", cfg.in_channels, H)
    return made


def test_flux_layout_roundtrip_and_load():
    cfg = F.tiny_flux()
    sd = _diffusers_state(cfg)
    orig = flux_diffusers_to_original(sd)
    assert is_flux_original(orig) and not is_flux_original(sd)
    H = cfg.hidden_size
    assert orig["double_blocks.0.img_attn.qkv.weight"].shape == (3 * H, H)
    assert orig["single_blocks.0.linear1.weight"].shape == (3 * H + cfg.mlp_dim, H)
    assert "final_layer.adaLN_modulation.1.weight" in orig and "double_blocks.0.txt_attn.norm.key_norm.scale" in orig
    # the AdaLN output order differs between the layouts: [shift; scale] vs [scale; shift]
    assert torch.equal(orig["final_layer.adaLN_modulation.1.weight"][:H], sd["norm_out.linear.weight"][H:])
    back = flux_original_to_diffusers({"model.diffusion_model." + k: v for k, v in orig.items()})
    assert set(back) == set(sd) and all(torch.equal(back[k], sd[k]) for k in sd)

    a = F.FluxTransformer(cfg, "cpu", get=lambda n: sd.get(n))
    b = F.FluxTransformer(cfg, "cpu", get=lambda n: back.get(n))
    g = torch.Generator().manual_seed(1)
    S_i, S_t = 16, 8
    img = torch.randn(1, S_i, cfg.in_channels, generator=g)
    txt = torch.randn(1, S_t, cfg.context_dim, generator=g)
    pooled = torch.randn(1, cfg.pooled_dim, generator=g)
    img_ids, txt_ids = F.flux_ids(4, 4, S_t)
    t = torch.tensor([0.7])
    gd = torch.tensor([3.5]) if cfg.guidance_embed else None
    ya = a.forward(img, txt, t, pooled, img_ids, txt_ids, gd)
    yb = b.forward(img, txt, t, pooled, img_ids, txt_ids, gd)
    assert torch.equal(ya, yb) and ya.float().abs().max() > 0


def test_image_service_merges_loras_into_a_flux_checkpoint(tmp_path, monkeypatch):
    """A PEFT-style adapter on a diffusers-layout transformer: the merged model differs from the base
    by exactly strength * (alpha / rank) * B A on the adapted weight."""
    from hartsyinference_b200.assets.safetensors import save_file
    from hartsyinference_b200.engine import InferenceEngine, ModelSpec
    from hartsyinference_b200.engine.requests import ImageRequest
    cfg = F.tiny_flux()
    monkeypatch.setattr(F, "FLUX_DEV", cfg)            # the service builds FLUX_DEV-shaped models from checkpoints
    sd = _diffusers_state(cfg)
    d = tmp_path / "flux"
    (d / "transformer").mkdir(parents=True)
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in sd.items()}, d / "transformer" / "model.safetensors")
    H = cfg.hidden_size
    g = torch.Generator().manual_seed(3)
    A, B = torch.randn(4, H, generator=g) * 0.3, torch.randn(H, 4, generator=g) * 0.3
    target = "transformer_blocks.0.attn.to_out.0"
    save_file({f"transformer.{target}.lora_A.weight": A, f"transformer.{target}.lora_B.weight": B,
               f"transformer.{target}.alpha": torch.tensor(8.0)}, tmp_path / "style.safetensors")
    eng = InferenceEngine("cpu")
    req = ImageRequest(prompt="x", width=32, height=32, steps=1, seed=1)
    base = eng.images.pipeline(ModelSpec(str(d)))
    tuned = eng.images.pipeline(ModelSpec(str(d)), ((str(tmp_path / "style.safetensors"), 0.5),))
    assert base is not tuned and len(eng.images.loaded_keys()) == 2
    wb = base.c.transformer.double[0][0].proj.weight.float()
    wt = tuned.c.transformer.double[0][0].proj.weight.float()
    want = 0.5 * (8.0 / 4) * (B @ A)
    assert torch.allclose(wt - wb, want, atol=0.05) and (wt - wb).abs().max() > 0.05
    assert torch.equal(base.c.transformer.double[1][0].proj.weight, tuned.c.transformer.double[1][0].proj.weight)
    res = eng.images.generate(ModelSpec(str(d)), ImageRequest(prompt="x", width=32, height=32, steps=1, seed=1,
                                                              loras=[(str(tmp_path / "style.safetensors"), 0.5)]))
    assert res.width == 32 and len(eng.images.loaded_keys()) == 2       # the cached merged pipeline is reused
    import pytest
    from hartsyinference_b200.exceptions import UnsupportedModelError
    with pytest.raises(UnsupportedModelError):
        eng.images.generate(ModelSpec("synthetic:flux-tiny"), ImageRequest(prompt="x", loras=[("a.safetensors", 1.0)]))
    eng.close()


def test_flux_directory_with_text_encoders(tmp_path, monkeypatch):
    """A diffusers-layout directory: transformer + CLIP text tower + T5 with their tokenizers. The
    prompt then conditions the image through the real encoders."""
    import json
    import pytest
    tr = pytest.importorskip("transformers")
    from hartsyinference_b200.assets.safetensors import save_file
    from hartsyinference_b200.assets.tokenizer import _bytes_to_unicode
    from hartsyinference_b200.engine import InferenceEngine, ModelSpec
    from hartsyinference_b200.engine.requests import ImageRequest
    cfg = F.tiny_flux(context_dim=64, pooled_dim=64)
    monkeypatch.setattr(F, "FLUX_DEV", cfg)
    d = tmp_path / "flux"
    (d / "transformer").mkdir(parents=True)
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in _diffusers_state(cfg).items()}, d / "transformer" / "model.safetensors")
    # CLIP text tower (pooled 64) with a byte-level vocabulary
    b2u = _bytes_to_unicode()
    vocab = {}
    for b in range(256):
        vocab[b2u[b]] = len(vocab)
    for b in range(256):
        vocab[b2u[b] + "</w>"] = len(vocab)
    vocab["<|startoftext|>"], vocab["<|endoftext|>"] = len(vocab), len(vocab) + 1
    hc = tr.CLIPTextConfig(vocab_size=len(vocab), hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=2,
                           max_position_embeddings=24, eos_token_id=len(vocab) - 1, bos_token_id=len(vocab) - 2, pad_token_id=len(vocab) - 1)
    torch.manual_seed(0)
    (d / "text_encoder").mkdir()
    (d / "tokenizer").mkdir()
    save_file({k: v.detach().contiguous() for k, v in tr.CLIPTextModel(hc).state_dict().items() if "position_ids" not in k},
              d / "text_encoder" / "model.safetensors")
    (d / "text_encoder" / "config.json").write_text(json.dumps(hc.to_dict()))
    (d / "tokenizer" / "vocab.json").write_text(json.dumps(vocab))
    (d / "tokenizer" / "merges.txt").write_text("#version: 0.2\n")
    # T5 encoder (d_model 64 = the transformer's context width) with a unigram vocabulary
    tc = tr.T5Config(vocab_size=40, d_model=64, d_kv=16, d_ff=128, num_layers=2, num_heads=4, feed_forward_proj="gated-gelu")
    (d / "text_encoder_2").mkdir()
    (d / "tokenizer_2").mkdir()
    save_file({k: v.detach().contiguous() for k, v in tr.T5EncoderModel(tc).state_dict().items()}, d / "text_encoder_2" / "model.safetensors")
    (d / "text_encoder_2" / "config.json").write_text(json.dumps(tc.to_dict()))
    pieces = [["<pad>", 0.0], ["</s>", 0.0], ["<unk>", 0.0], ["▁", -2.0]] + [[ch, -3.0 - i * 0.01] for i, ch in enumerate("abcdefghijklmnopqrstuvwxyz")]
    (d / "tokenizer_2" / "tokenizer.json").write_text(json.dumps({
        "model": {"type": "Unigram", "unk_id": 2, "vocab": pieces},
        "added_tokens": [{"id": 0, "content": "<pad>", "special": True}, {"id": 1, "content": "</s>", "special": True},
                         {"id": 2, "content": "<unk>", "special": True}]}))
    eng = InferenceEngine("cpu")
    pipe = eng.images.pipeline(ModelSpec(str(d)))
    assert pipe.c.t5 is not None and pipe.c.clip is not None
    ctx_a, pooled_a = pipe.encode_prompt("a red fox", max_len=16)
    ctx_b, pooled_b = pipe.encode_prompt("a blue whale", max_len=16)
    assert ctx_a.shape == (16, 64) and pooled_a.shape == (64,)
    assert not torch.allclose(ctx_a.float(), ctx_b.float()) and not torch.allclose(pooled_a.float(), pooled_b.float())
    assert torch.equal(ctx_a, pipe.encode_prompt("a red fox", max_len=16)[0])
    res = eng.images.generate(ModelSpec(str(d)), ImageRequest(prompt="a red fox", width=32, height=32, steps=1, seed=1))
    assert (res.width, res.height) == (32, 32)
    eng.close()


def test_weighted_prompt_reaches_the_t5_states():
    """With a T5 stack loaded, ``(word:w)`` scales that word's token states and leaves the plain text otherwise."""
    import pytest
    tr = pytest.importorskip("transformers")
    from hartsyinference_b200.assets.tokenizer import UnigramTokenizer
    from hartsyinference_b200.models.encoders.t5 import T5Config, T5Encoder
    from hartsyinference_b200.pipelines.flux import FluxComponents, FluxPipeline
    cfg = F.tiny_flux(context_dim=64, pooled_dim=32)
    pieces = [("<pad>", 0.0), ("</s>", 0.0), ("<unk>", 0.0), ("▁", -2.0)] + [(ch, -3.0) for ch in "abcdefghijklmnopqrstuvwxyz"]
    tok = UnigramTokenizer(pieces, unk_id=2, eos_id=1, specials={"<pad>": 0, "</s>": 1, "<unk>": 2})
    t5 = T5Encoder(T5Config(vocab_size=40, d_model=64, d_kv=16, d_ff=128, num_layers=1, num_heads=4), "cpu", seed=1)
    pipe = FluxPipeline(FluxComponents(F.FluxTransformer(cfg, "cpu", seed=0), t5=t5, t5_tokenizer=tok))
    plain, _ = pipe.encode_prompt("a red fox", max_len=24)
    same, _ = pipe.encode_prompt("a (red:1.0) fox", max_len=24)
    heavy, _ = pipe.encode_prompt("a (red:2.0) fox", max_len=24)
    assert plain.shape == heavy.shape == (24, 64)
    assert not torch.allclose(plain.float(), heavy.float(), atol=1e-3)
    # the weighted and the plain prompt tokenise to the same pieces here, so weight 1.0 changes nothing
    assert torch.allclose(plain.float(), same.float(), atol=1e-2)
