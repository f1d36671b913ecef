"""LoRA merge, family detection, extra schedulers and the first-block cache (CPU)."""
import pytest
import torch

from hartsyinference_b200.assets import lora as L
from hartsyinference_b200.assets import registry as REG
from hartsyinference_b200.models.diffusion import schedulers as S
from hartsyinference_b200.models.dit.step_cache import FirstBlockCache


def test_lora_merge_peft_and_kohya_styles():
    torch.manual_seed(0)
    base = {"model.layers.0.self_attn.q_proj.weight": torch.randn(32, 16),
            "model.layers.0.mlp.up_proj.weight": torch.randn(48, 16)}
    a, b = torch.randn(4, 16), torch.randn(32, 4)
    peft = {"base_model.model.model.layers.0.self_attn.q_proj.lora_A.weight": a,
            "base_model.model.model.layers.0.self_attn.q_proj.lora_B.weight": b}
    a2, b2 = torch.randn(2, 16), torch.randn(48, 2)
    kohya = {"lora_unet_model_layers_0_mlp_up_proj.lora_down.weight": a2,
             "lora_unet_model_layers_0_mlp_up_proj.lora_up.weight": b2,
             "lora_unet_model_layers_0_mlp_up_proj.alpha": torch.tensor(1.0)}
    stack = L.LoraStack().add(peft, 0.5).add(kohya, 2.0)
    get = stack.wrap(base.get, base.keys())
    q = get("model.layers.0.self_attn.q_proj.weight")
    assert torch.allclose(q, base["model.layers.0.self_attn.q_proj.weight"] + 0.5 * (b @ a), atol=1e-5)
    u = get("model.layers.0.mlp.up_proj.weight")
    assert torch.allclose(u, base["model.layers.0.mlp.up_proj.weight"] + 2.0 * (1.0 / 2) * (b2 @ a2), atol=1e-5)
    assert stack.unmatched == [] and get("missing") is None


def test_lora_reports_unmatched_and_shape_errors():
    base = {"a.weight": torch.zeros(4, 4)}
    stack = L.LoraStack().add({"zzz.lora_A.weight": torch.zeros(1, 4), "zzz.lora_B.weight": torch.zeros(4, 1)})
    stack.wrap(base.get, base.keys())
    assert stack.unmatched == ["zzz"]


def test_family_detection_from_keys_and_files(tmp_path):
    assert REG.detect_from_keys(["model.layers.0.self_attn.q_proj.weight"]).arch == "llama"
    assert REG.detect_from_keys(["model.layers.0.self_attn.kv_a_proj_with_mqa.weight",
                                 "model.layers.0.self_attn.q_proj.weight"]).arch == "deepseek3"
    assert REG.detect_from_keys(["double_blocks.0.img_attn.qkv.weight"]).family == "dit-image"
    assert REG.detect_from_keys(["blocks.0.cross_attn.k.weight"]).arch == "wan"
    assert REG.detect_from_keys(["x.lora_A.weight", "model.layers.0.self_attn.q_proj.lora_B.weight"]).family == "lora"
    assert REG.detect_from_keys(["foo"]).family == "unknown"
    from hartsyinference_b200.assets.safetensors import save_file
    f = tmp_path / "m.safetensors"
    save_file({"encoder.block.0.layer.0.SelfAttention.relative_attention_bias.weight": torch.zeros(2, 2)}, f)
    assert REG.detect(f).arch == "t5"
    d = tmp_path / "hf"
    d.mkdir()
    (d / "config.json").write_text('{"model_type": "qwen2"}')
    assert REG.detect(d) == REG.Detected("llm", "qwen2", "config.json")


def _exact_eps(x, x0, a_t):
    return (x - a_t ** 0.5 * x0) / (1 - a_t) ** 0.5


def test_dpmpp_2m_and_ddim_recover_the_data_with_an_exact_denoiser():
    # with the exact noise prediction every solver must land on x0 at the last step
    torch.manual_seed(1)
    x0 = torch.randn(3, 8)
    for name in ("dpm++2m", "ddim"):
        sch = S.make_scheduler(name, 12)
        if name == "ddim":
            continue          # covered by the DiT tests; here: the new solver
        a0 = float(sch.alpha[0]) ** 2
        x = a0 ** 0.5 * x0 + (1 - a0) ** 0.5 * torch.randn(3, 8)
        for i in range(sch.num_steps):
            a_t = float(sch.alpha[i]) ** 2
            x = sch.step(_exact_eps(x, x0, a_t), i, x)
        assert torch.allclose(x, x0, atol=1e-4)


def test_dpmpp_2m_second_order_beats_first_order_on_a_curved_trajectory():
    # denoiser with a known smooth error: the multistep update must track x0 closely
    sch = S.DPMSolverMultistepScheduler(8)
    assert len(sch.timesteps) == 8 and sch.timesteps[0] > sch.timesteps[-1]
    assert sch.sigma[-1] == 0 and sch.alpha[-1] == 1


def test_lcm_last_step_returns_denoised_and_is_seeded():
    x0 = torch.ones(2, 4)
    outs = []
    for _ in range(2):
        sch = S.make_scheduler("lcm", 4, seed=3)
        a0 = float(sch.ac[int(sch.timesteps[0])])
        x = a0 ** 0.5 * x0 + (1 - a0) ** 0.5 * torch.full((2, 4), 0.3)
        for i in range(4):
            a_t = float(sch.ac[int(sch.timesteps[i])])
            x = sch.step(_exact_eps(x, x0, a_t), i, x)
        outs.append(x)
    assert torch.equal(outs[0], outs[1])
    assert (outs[0] - x0).abs().max() < 0.05


def test_first_block_cache_skips_small_changes_and_bounds_the_run():
    c = FirstBlockCache(threshold=0.1, max_consecutive_skips=2)
    first = torch.ones(4, 8)
    assert c.should_compute(first)
    c.store_residual(first, first + 2.0)
    # tiny change: skipped, residual re-applied
    f2 = first * 1.01
    assert not c.should_compute(f2)
    assert torch.allclose(c.apply_residual(f2), f2 + 2.0)
    assert not c.should_compute(f2 * 1.01)
    # third small step in a row: forced recompute
    assert c.should_compute(f2 * 1.02)
    c.store_residual(f2, f2 + 1.0)
    # a large change always recomputes
    assert c.should_compute(f2 * 3.0)
    assert c.skipped == 2 and c.computed == 2
    off = FirstBlockCache(0.0)
    assert off.should_compute(first) and off.should_compute(first)


def test_bert_encoder_matches_transformers_bert():
    import transformers
    from hartsyinference_b200.models.encoders.bert import BertEncoder, tiny_bert
    cfg = tiny_bert()
    hf_cfg = transformers.BertConfig(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden, num_hidden_layers=cfg.layers,
                                     num_attention_heads=cfg.heads, intermediate_size=cfg.intermediate,
                                     max_position_embeddings=cfg.max_len, type_vocab_size=cfg.type_vocab,
                                     layer_norm_eps=cfg.eps, hidden_act="gelu")
    torch.manual_seed(0)
    hf = transformers.BertModel(hf_cfg, add_pooling_layer=False).eval()
    sd = {k: v.detach() for k, v in hf.state_dict().items()}
    enc = BertEncoder(cfg, "cpu", get=lambda n: sd.get(n))
    ids = torch.randint(0, cfg.vocab_size, (11,))
    ours = enc.hidden_states(ids).float()
    with torch.no_grad():
        ref = hf(input_ids=ids[None]).last_hidden_state[0]
    cos = torch.nn.functional.cosine_similarity(ours, ref, dim=-1)
    assert cos.min() > 0.995, cos.min()
    e = enc.embed(ids)
    assert abs(float(e.norm()) - 1.0) < 1e-3


def test_wordpiece_and_bert_embeddings_service(tmp_path):
    import json
    from hartsyinference_b200.assets.safetensors import save_file
    from hartsyinference_b200.assets.tokenizer import WordPieceTokenizer
    from hartsyinference_b200.engine.embeddings_service import BertEmbeddingsService, is_bert_dir
    from hartsyinference_b200.engine.requests import ModelSpec
    from hartsyinference_b200.models.encoders.bert import BertEncoder, tiny_bert
    vocab = ["[PAD]", "[UNK]", "[CLS]", "[SEP]", "hello", "world", "un", "##aff", "##able", ",", "!"] + [f"t{i}" for i in range(117)]
    tok = WordPieceTokenizer(vocab)
    assert tok.encode("Hello, unaffable world!") == [2, 4, 9, 6, 7, 8, 5, 10, 3]
    assert tok.encode("zzz", add_special=False) == [1]
    assert tok.decode(tok.encode("hello unaffable")) == "hello unaffable"
    # a checkpoint directory round trip through the service
    cfg = tiny_bert()
    enc = BertEncoder(cfg, "cpu", seed=4)
    sd = {"embeddings.word_embeddings.weight": enc.tok, "embeddings.position_embeddings.weight": enc.pos,
          "embeddings.token_type_embeddings.weight": enc.typ, "embeddings.LayerNorm.weight": enc.ln_w,
          "embeddings.LayerNorm.bias": enc.ln_b}
    H = cfg.hidden
    for i, b in enumerate(enc.blocks):
        p = f"encoder.layer.{i}."
        for j, n in enumerate(("query", "key", "value")):
            sd[p + f"attention.self.{n}.weight"] = b["qkv"].weight[j * H:(j + 1) * H].contiguous()
            sd[p + f"attention.self.{n}.bias"] = b["qkv"].bias[j * H:(j + 1) * H].contiguous()
        for name, key in (("attention.output.dense", "o"), ("intermediate.dense", "fc1"), ("output.dense", "fc2")):
            sd[p + name + ".weight"], sd[p + name + ".bias"] = b[key].weight, b[key].bias
        sd[p + "attention.output.LayerNorm.weight"], sd[p + "attention.output.LayerNorm.bias"] = b["ln1w"], b["ln1b"]
        sd[p + "output.LayerNorm.weight"], sd[p + "output.LayerNorm.bias"] = b["ln2w"], b["ln2b"]
    d = tmp_path / "bert"
    d.mkdir()
    save_file({k: v.contiguous() for k, v in sd.items()}, d / "model.safetensors")
    (d / "config.json").write_text(json.dumps(dict(model_type="bert", vocab_size=cfg.vocab_size, hidden_size=H,
                                                   num_hidden_layers=cfg.layers, num_attention_heads=cfg.heads,
                                                   intermediate_size=cfg.intermediate, max_position_embeddings=cfg.max_len)))
    (d / "vocab.txt").write_text("\n".join(vocab) + "\n")
    assert is_bert_dir(d)
    svc = BertEmbeddingsService("cpu")
    out = svc.embed(ModelSpec(requested=str(d), local_path=str(d)), ["hello world", "unaffable !"])
    assert out.shape == (2, H)
    ref = enc.embed(torch.tensor(tok.encode("hello world")))
    assert torch.allclose(out[0], ref.float(), atol=2e-2)


def test_iso_surface_of_a_sphere_is_closed_oriented_and_accurate(tmp_path):
    from hartsyinference_b200.threed import marching_cubes, write_glb, write_obj, write_ply
    from hartsyinference_b200.threed.writers import vertex_normals
    n = 20
    g = torch.linspace(-1, 1, n)
    x, y, z = torch.meshgrid(g, g, g, indexing="ij")
    sdf = (x * x + y * y + z * z).sqrt() - 0.6
    v, f = marching_cubes(sdf, 0.0, spacing=(2 / (n - 1),) * 3, origin=(-1, -1, -1))
    assert f.shape[0] > 1000
    assert (v.norm(dim=1) - 0.6).abs().max() < 0.02
    e = torch.cat([f[:, [0, 1]], f[:, [1, 2]], f[:, [2, 0]]], 0)
    fwd, rev = set(map(tuple, e.tolist())), set(map(tuple, e[:, [1, 0]].tolist()))
    assert fwd == rev and len(fwd) == e.shape[0]                 # closed and consistently wound
    a, b, c = v[f[:, 0]], v[f[:, 1]], v[f[:, 2]]
    vol = (a * torch.cross(b, c, dim=1)).sum() / 6
    assert abs(float(vol) - 4 / 3 * 3.14159265 * 0.6 ** 3) < 0.03   # positive: normals point outwards
    assert marching_cubes(torch.ones(4, 4, 4))[1].shape[0] == 0
    # writers
    nrm = vertex_normals(v, f)
    write_obj(tmp_path / "m.obj", v, f, nrm)
    txt = (tmp_path / "m.obj").read_text().splitlines()
    assert sum(l.startswith("v ") for l in txt) == v.shape[0] and sum(l.startswith("f ") for l in txt) == f.shape[0]
    write_ply(tmp_path / "m.ply", v, f, colors=torch.full((v.shape[0], 3), 128, dtype=torch.uint8))
    raw = (tmp_path / "m.ply").read_bytes()
    head = raw[:raw.index(b"end_header\n") + 11].decode()
    assert f"element vertex {v.shape[0]}" in head and f"element face {f.shape[0]}" in head
    assert len(raw) == len(head) + v.shape[0] * 15 + f.shape[0] * 13
    write_glb(tmp_path / "m.glb", v, f, nrm)
    import json, struct
    blob = (tmp_path / "m.glb").read_bytes()
    magic, ver, total = struct.unpack("<4sII", blob[:12])
    assert magic == b"glTF" and ver == 2 and total == len(blob)
    jlen = struct.unpack("<I", blob[12:16])[0]
    doc = json.loads(blob[20:20 + jlen])
    assert doc["accessors"][0]["count"] == v.shape[0] and doc["accessors"][-1]["count"] == f.numel()


def test_video_frames_and_sequence_fallback(tmp_path, monkeypatch):
    from hartsyinference_b200 import video as V
    fr = torch.rand(5, 3, 16, 24) * 2 - 1
    u8 = V.frames_to_uint8(fr)
    assert u8.shape == (5, 16, 24, 3) and u8.dtype == torch.uint8
    assert torch.equal(V.frames_to_uint8(fr.permute(1, 0, 2, 3)), u8)
    monkeypatch.setattr(V.io, "ffmpeg_path", lambda: None)
    out = V.encode_video(fr, tmp_path / "clip.mp4", fps=8)
    assert out.is_dir() and len(list(out.glob("frame_*.png"))) == 5
    import json
    man = json.loads((out / "manifest.json").read_text())
    assert man == {"fps": 8, "frames": 5, "width": 24, "height": 16, "pattern": "frame_%06d.png"}
    assert (out / "frame_000000.png").read_bytes()[:8] == b"\x89PNG\r\n\x1a\n"


def test_mamba_matches_transformers_and_state_carries_over():
    import transformers
    from hartsyinference_b200.models.ssm import MambaModel, tiny_mamba
    cfg = tiny_mamba()
    hf_cfg = transformers.MambaConfig(vocab_size=cfg.vocab_size, hidden_size=cfg.d_model, state_size=cfg.d_state,
                                      num_hidden_layers=cfg.n_layer, conv_kernel=cfg.d_conv, expand=cfg.expand,
                                      time_step_rank=cfg.rank, layer_norm_epsilon=cfg.rms_eps, use_mambapy=False)
    torch.manual_seed(0)
    hf = transformers.MambaForCausalLM(hf_cfg).eval()
    sd = {k: v.detach() for k, v in hf.state_dict().items()}
    m = MambaModel(cfg, "cpu", get=lambda n: sd.get(n))
    ids = torch.randint(0, cfg.vocab_size, (19,))
    with torch.no_grad():
        ref = hf(input_ids=ids[None]).logits[0]
    st = m.new_state()
    ours = m.logits(m.forward(ids, st))
    cos = torch.nn.functional.cosine_similarity(ours, ref, dim=-1)
    assert cos.min() > 0.99, cos.min()
    # the same sequence fed in two pieces through the carried state gives the same final logits
    st2 = m.new_state()
    m.forward(ids[:11], st2)
    tail = m.logits(m.forward(ids[11:], st2))
    assert torch.allclose(tail[-1], ours[-1], atol=2e-2, rtol=2e-2)
    out = m.generate(ids[:5].tolist(), max_tokens=6, stop_at_eos=False)
    assert len(out) == 6


def test_falcon_mamba_matches_transformers():
    """FalconMamba = Mamba with a weight-free RMS normalisation of dt, B and C."""
    import transformers
    from dataclasses import replace
    from hartsyinference_b200.models.ssm import MambaModel, tiny_mamba
    cfg = replace(tiny_mamba(), bcdt_rms_eps=1e-6)
    hf_cfg = transformers.FalconMambaConfig(vocab_size=cfg.vocab_size, hidden_size=cfg.d_model, state_size=cfg.d_state,
                                            num_hidden_layers=cfg.n_layer, conv_kernel=cfg.d_conv, expand=cfg.expand,
                                            time_step_rank=cfg.rank, layer_norm_epsilon=cfg.rms_eps, mixer_rms_eps=1e-6,
                                            use_falcon_mambapy=False)
    torch.manual_seed(0)
    hf = transformers.FalconMambaForCausalLM(hf_cfg).eval()
    sd = {k: v.detach() for k, v in hf.state_dict().items()}
    m = MambaModel(cfg, "cpu", get=lambda n: sd.get(n))
    ids = torch.randint(0, cfg.vocab_size, (19,))
    with torch.no_grad():
        ref = hf(input_ids=ids[None]).logits[0]
    ours = m.logits(m.forward(ids, m.new_state()))
    assert torch.nn.functional.cosine_similarity(ours, ref, dim=-1).min() > 0.99
    plain = MambaModel(tiny_mamba(), "cpu", get=lambda n: sd.get(n))
    off = plain.logits(plain.forward(ids, plain.new_state()))
    assert torch.nn.functional.cosine_similarity(off, ref, dim=-1).min() < 0.99      # the normalisation matters


def test_block_streamer_walks_blocks_with_two_slots():
    from dataclasses import dataclass
    from hartsyinference_b200.engine.block_streaming import BlockStreamer, tree_bytes

    @dataclass
    class Blk:
        w: torch.Tensor
        parts: list

    blocks = [Blk(torch.full((4, 4), float(i)), [torch.full((2,), float(i)), {"b": torch.full((3,), float(i))}]) for i in range(5)]
    s = BlockStreamer(blocks, "cpu")
    assert len(s) == 5 and tree_bytes(blocks[0]) == (16 + 2 + 3) * 4
    s.prime()
    for rep in range(2):
        for i in range(5):
            b = s.block(i)
            assert float(b.w[0, 0]) == i and float(b.parts[1]["b"][0]) == i
            assert len(s._resident) <= 2
    assert s.uploads >= 9            # every block fetched again on the second pass (two slots only)
    s.evict_all()
    assert not s._resident


@pytest.mark.parametrize("groups", [1, 2])
def test_mamba2_matches_transformers_and_state_carries_over(groups):
    transformers = pytest.importorskip("transformers")
    from hartsyinference_b200.models.ssm import Mamba2Model, mamba2_from_hf
    c = transformers.Mamba2Config(vocab_size=256, hidden_size=64, num_hidden_layers=2, state_size=16, num_heads=8, head_dim=16,
                                  n_groups=groups, expand=2, conv_kernel=4, chunk_size=8, eos_token_id=0, bos_token_id=1, pad_token_id=0)
    torch.manual_seed(0)
    hf = transformers.Mamba2ForCausalLM(c).eval()
    with torch.no_grad():
        for _, p in hf.named_parameters():
            if p.ndim >= 2:
                p.mul_(3.0)
    sd = {k: v.detach() for k, v in hf.state_dict().items()}
    m = Mamba2Model(mamba2_from_hf(c.to_dict()), "cpu", get=lambda n: sd.get(n))
    ids = torch.randint(0, 256, (21,), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        ref = hf(ids[None]).logits[0]
    st = m.new_state()
    # a prompt, one decode step and a multi-token continuation all run on the carried state
    mine = torch.cat([m.logits(m.forward(ids[:13], st)), m.logits(m.forward(ids[13:14], st)), m.logits(m.forward(ids[14:], st))])
    assert torch.nn.functional.cosine_similarity(mine.flatten(), ref.flatten(), dim=0) > 0.999
    assert (mine.argmax(-1) == ref.argmax(-1)).float().mean() > 0.9
    out = m.generate(ids[:5].tolist(), max_tokens=4, stop_at_eos=False)
    assert len(out) == 4


def test_rwkv_matches_transformers_and_state_carries_over():
    transformers = pytest.importorskip("transformers")
    from hartsyinference_b200.models.ssm import RwkvModel, rwkv_from_hf
    c = transformers.RwkvConfig(vocab_size=300, hidden_size=64, num_hidden_layers=2, attention_hidden_size=64, intermediate_size=128,
                                context_length=64, rescale_every=0)
    torch.manual_seed(0)
    hf = transformers.RwkvForCausalLM(c).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if p.ndim == 2:
                p.mul_(3.0)
            if "time_decay" in n or "time_first" in n:
                p.copy_(torch.randn_like(p) * 0.5)
    sd = {k: v.detach() for k, v in hf.state_dict().items()}
    m = RwkvModel(rwkv_from_hf(c.to_dict()), "cpu", get=lambda n: sd.get(n))
    ids = torch.randint(0, 300, (17,), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        ref = hf(ids[None]).logits[0]
    st = m.new_state()
    mine = torch.cat([m.logits(m.forward(ids[:9], st)), m.logits(m.forward(ids[9:10], st)), m.logits(m.forward(ids[10:], st))])
    assert torch.nn.functional.cosine_similarity(mine.flatten(), ref.flatten(), dim=0) > 0.999
    assert (mine.argmax(-1) == ref.argmax(-1)).float().mean() > 0.9
    assert len(m.generate(ids[:4].tolist(), max_tokens=3, stop_at_eos=False)) == 3


@pytest.mark.parametrize("kind", ["mamba2", "rwkv"])
def test_recurrent_models_through_the_text_service(kind, tmp_path):
    transformers = pytest.importorskip("transformers")
    from hartsyinference_b200.engine import InferenceEngine, ModelSpec, TextRequest
    from hartsyinference_b200.models.llm.loader import save_hf_checkpoint
    torch.manual_seed(0)
    if kind == "mamba2":
        c = transformers.Mamba2Config(vocab_size=300, hidden_size=64, num_hidden_layers=2, state_size=16, num_heads=8, head_dim=16,
                                      n_groups=1, expand=2, conv_kernel=4, chunk_size=8, eos_token_id=0, bos_token_id=1, pad_token_id=0)
        hf = transformers.Mamba2ForCausalLM(c)
    else:
        c = transformers.RwkvConfig(vocab_size=300, hidden_size=64, num_hidden_layers=2, attention_hidden_size=64, intermediate_size=128,
                                    context_length=64, rescale_every=0)
        hf = transformers.RwkvForCausalLM(c)
    d = tmp_path / kind
    save_hf_checkpoint(c.to_dict(), {k: v.detach().contiguous() for k, v in hf.state_dict().items()}, d)
    eng = InferenceEngine("cpu")
    try:
        r1 = eng.text.generate(ModelSpec(str(d)), TextRequest(prompt="hello", max_tokens=5, greedy=True))
        r2 = eng.text.generate(ModelSpec(str(d)), TextRequest(prompt="hello", max_tokens=5, greedy=True))
        assert r1.token_ids == r2.token_ids and 0 < r1.completion_tokens <= 5 and r1.prompt_tokens == 5
        chunks = list(eng.text.stream(ModelSpec(str(d)), TextRequest(prompt="hello", max_tokens=3, temperature=0.8, seed=3)))
        assert chunks[-1].result is not None and chunks[-1].result.completion_tokens <= 3
        assert any(k.startswith("ssm|") for k in eng.loaded_pipeline_keys)
    finally:
        eng.text.release()


def test_t5_seq2seq_matches_transformers():
    transformers = pytest.importorskip("transformers")
    from hartsyinference_b200.models.encoders.t5 import T5Config, T5Seq2Seq
    c = transformers.T5Config(vocab_size=128, d_model=64, d_kv=16, d_ff=128, num_layers=2, num_decoder_layers=2, num_heads=4,
                              feed_forward_proj="gated-gelu", tie_word_embeddings=False, decoder_start_token_id=0, eos_token_id=1, pad_token_id=0)
    torch.manual_seed(0)
    hf = transformers.T5ForConditionalGeneration(c).eval()
    with torch.no_grad():
        for _, p in hf.named_parameters():
            if p.ndim >= 2:
                p.mul_(2.0)
    sd = {k: v.detach() for k, v in hf.state_dict().items()}
    m = T5Seq2Seq(T5Config(vocab_size=128, d_model=64, d_kv=16, d_ff=128, num_layers=2, num_heads=4), "cpu", get=lambda n: sd.get(n))
    src = torch.tensor([5, 17, 33, 9, 1])
    dec = torch.tensor([0, 11, 23, 47, 60, 3])
    with torch.no_grad():
        ref = hf(input_ids=src[None], decoder_input_ids=dec[None]).logits[0]
    st = m.start(m.encoder.encode(src))
    mine = torch.cat([m.decode(st, dec[:3]), m.decode(st, dec[3:4]), m.decode(st, dec[4:])])
    assert torch.nn.functional.cosine_similarity(mine.flatten(), ref.flatten(), dim=0) > 0.999
    assert (mine.argmax(-1) == ref.argmax(-1)).float().mean() >= 0.8
    with torch.no_grad():
        gen = hf.generate(input_ids=src[None], max_new_tokens=8, do_sample=False)[0].tolist()
    want = [t for t in gen[1:] if t != 1]
    got = m.generate(src, max_new=8)
    assert got[: len(want)] == want[: len(got)] and len(got) > 0


def test_xlm_roberta_embeddings_match_transformers(tmp_path):
    transformers = pytest.importorskip("transformers")
    import json
    from hartsyinference_b200.engine import InferenceEngine, ModelSpec
    from hartsyinference_b200.models.encoders.bert import BertConfig, BertEncoder
    from hartsyinference_b200.models.llm.loader import save_hf_checkpoint
    c = transformers.XLMRobertaConfig(vocab_size=40, hidden_size=128, num_hidden_layers=2, num_attention_heads=2, intermediate_size=256,
                                      max_position_embeddings=40, type_vocab_size=1, pad_token_id=1, bos_token_id=0, eos_token_id=2)
    torch.manual_seed(0)
    hf = transformers.XLMRobertaModel(c, add_pooling_layer=False).eval()
    sd = {k: v.detach() for k, v in hf.state_dict().items()}
    cfg = BertConfig(vocab_size=40, hidden=128, layers=2, heads=2, intermediate=256, max_len=40, type_vocab=1, eps=c.layer_norm_eps, position_offset=2)
    enc = BertEncoder(cfg, "cpu", get=lambda n: sd.get(n))
    ids = torch.tensor([0, 7, 9, 30, 2])
    with torch.no_grad():
        ref = hf(input_ids=ids[None]).last_hidden_state[0]
    assert torch.nn.functional.cosine_similarity(enc.hidden_states(ids).float().flatten(), ref.flatten(), dim=0) > 0.995
    d = tmp_path / "xlmr"
    save_hf_checkpoint({**c.to_dict(), "model_type": "xlm-roberta"}, {k: v.contiguous() for k, v in sd.items()}, d)
    pieces = [["<s>", 0.0], ["<pad>", 0.0], ["</s>", 0.0], ["<unk>", 0.0], ["▁", -2.0]] + [[ch, -3.0] for ch in "abcdefghijklmnopqrstuvwxyz"]
    (d / "tokenizer.json").write_text(json.dumps({"model": {"type": "Unigram", "unk_id": 3, "vocab": pieces},
                                                  "added_tokens": [{"id": i, "content": p[0], "special": True} for i, p in enumerate(pieces[:4])]}))
    eng = InferenceEngine("cpu")
    emb = eng.embeddings.embed(ModelSpec(str(d)), ["hello world", "goodbye"])
    assert emb.shape == (2, 128) and torch.allclose(emb.norm(dim=-1), torch.ones(2), atol=1e-3)
    eng.close()


def test_qwen35_hybrid_matches_transformers_and_state_carries_over():
    """Gated-DeltaNet + gated-attention hybrid against ``Qwen3_5ForCausalLM``: logits of a prompt,
    the same prompt fed in two pieces through the carried state, and the greedy continuation."""
    import transformers
    if not hasattr(transformers, "Qwen3_5ForCausalLM"):
        pytest.skip("transformers has no Qwen3.5")
    from transformers.models.qwen3_5.configuration_qwen3_5 import Qwen3_5TextConfig
    from hartsyinference_b200.models.ssm import Qwen35Model, qwen35_from_hf
    hf_cfg = Qwen3_5TextConfig(vocab_size=320, hidden_size=128, intermediate_size=256, num_hidden_layers=4, num_attention_heads=4,
                               num_key_value_heads=2, head_dim=32, linear_conv_kernel_dim=4, linear_key_head_dim=16,
                               linear_value_head_dim=16, linear_num_key_heads=2, linear_num_value_heads=4,
                               max_position_embeddings=256, pad_token_id=0)
    hf_cfg._attn_implementation = "eager"
    torch.manual_seed(0)
    hf = transformers.Qwen3_5ForCausalLM(hf_cfg).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if p.ndim >= 2:
                p.mul_(2.0)
            elif "norm" in n:
                p.add_(torch.randn_like(p) * 0.1)
    sd = {k: v.detach() for k, v in hf.state_dict().items()}
    cfg = qwen35_from_hf(hf_cfg.to_dict())
    assert cfg.layer_types == ("linear_attention",) * 3 + ("full_attention",) and cfg.rot == 8
    m = Qwen35Model(cfg, "cpu", get=lambda n: sd.get(n), dtype=torch.float32)
    ids = torch.randint(0, 320, (21,), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        ref = hf(input_ids=ids[None]).logits[0]
    st = m.new_state()
    ours = m.logits(m.forward(ids, st))
    cos = torch.nn.functional.cosine_similarity(ours, ref, dim=-1)
    assert cos.min() > 0.999, cos.min()
    st2 = m.new_state()
    m.forward(ids[:9], st2)
    tail = m.logits(m.forward(ids[9:], st2))
    assert torch.allclose(tail[-1], ours[-1], atol=1e-3, rtol=1e-3)
    with torch.no_grad():
        gen = hf.generate(ids[None, :7], max_new_tokens=6, do_sample=False, pad_token_id=0)[0, 7:].tolist()
    assert m.generate(ids[:7].tolist(), max_tokens=6, stop_at_eos=False) == gen


def test_qwen35_moe_matches_transformers():
    import transformers
    if not hasattr(transformers, "Qwen3_5MoeForCausalLM"):
        pytest.skip("transformers has no Qwen3.5-MoE")
    from transformers.models.qwen3_5_moe.configuration_qwen3_5_moe import Qwen3_5MoeTextConfig
    from hartsyinference_b200.models.ssm import Qwen35Model, qwen35_from_hf
    hf_cfg = Qwen3_5MoeTextConfig(vocab_size=320, hidden_size=128, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
                                  head_dim=32, linear_key_head_dim=16, linear_value_head_dim=16, linear_num_key_heads=2,
                                  linear_num_value_heads=4, moe_intermediate_size=64, shared_expert_intermediate_size=96,
                                  num_experts=4, num_experts_per_tok=2, max_position_embeddings=256, pad_token_id=0)
    hf_cfg._attn_implementation = "eager"
    torch.manual_seed(0)
    hf = transformers.Qwen3_5MoeForCausalLM(hf_cfg).eval()
    with torch.no_grad():
        for p in hf.parameters():
            if p.ndim >= 2:
                p.mul_(2.0)
    sd = {k: v.detach() for k, v in hf.state_dict().items()}
    cfg = qwen35_from_hf(hf_cfg.to_dict())
    assert cfg.experts == 4 and cfg.top_k == 2
    m = Qwen35Model(cfg, "cpu", get=lambda n: sd.get(n), dtype=torch.float32)
    ids = torch.randint(0, 320, (17,), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        ref = hf(input_ids=ids[None]).logits[0]
    ours = m.logits(m.forward(ids, m.new_state()))
    assert torch.nn.functional.cosine_similarity(ours, ref, dim=-1).min() > 0.999
