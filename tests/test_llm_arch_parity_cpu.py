"""Every decoder architecture the config factory claims, checked against transformers: a tiny
random model of that family is saved as a checkpoint directory, loaded through ``load_llm`` and its
prefill logits are compared with the Hugging Face forward of the same weights."""
import pytest
import torch

from hartsyinference_b200.models.llm.loader import load_llm, save_hf_checkpoint
from hartsyinference_b200.models.llm.transformer import ForwardBatch

tr = pytest.importorskip("transformers")

_BASE = dict(vocab_size=320, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
             num_key_value_heads=2, max_position_embeddings=256)

ARCHS = {
    "llama": ("LlamaConfig", dict(rope_theta=10000.0)),
    "llama3_rope": ("LlamaConfig", dict(rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                                       "high_freq_factor": 4.0, "original_max_position_embeddings": 64})),
    "mistral": ("MistralConfig", dict(sliding_window=None)),
    "qwen2": ("Qwen2Config", dict()),
    "qwen3": ("Qwen3Config", dict(head_dim=32)),
    "gemma": ("GemmaConfig", dict(head_dim=32)),
    "gemma2": ("Gemma2Config", dict(head_dim=32, sliding_window=8, query_pre_attn_scalar=32)),
    "gemma3_text": ("Gemma3TextConfig", dict(head_dim=32, sliding_window=8, query_pre_attn_scalar=32)),
    "granite": ("GraniteConfig", dict(residual_multiplier=0.5, embedding_multiplier=3.0, logits_scaling=2.0,
                                      attention_multiplier=0.2)),
    "olmo2": ("Olmo2Config", dict()),
    "mixtral": ("MixtralConfig", dict(num_local_experts=4, num_experts_per_tok=2)),
    "qwen2_moe": ("Qwen2MoeConfig", dict(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=64,
                                         shared_expert_intermediate_size=128, decoder_sparse_step=1, mlp_only_layers=[])),
    "qwen3_moe": ("Qwen3MoeConfig", dict(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=64, head_dim=32,
                                         decoder_sparse_step=1, mlp_only_layers=[], norm_topk_prob=True)),
    "olmoe": ("OlmoeConfig", dict(num_experts=4, num_experts_per_tok=2)),
    "phi3": ("Phi3Config", dict(pad_token_id=0)),
    "glm": ("GlmConfig", dict(head_dim=32, pad_token_id=0)),
    "glm4": ("Glm4Config", dict(head_dim=32, pad_token_id=0)),
    "starcoder2": ("Starcoder2Config", dict()),
    "stablelm": ("StableLmConfig", dict()),
    "stablelm_parallel": ("StableLmConfig", dict(use_parallel_residual=True, use_qkv_bias=True)),
    "cohere": ("CohereConfig", dict()),
    "cohere2": ("Cohere2Config", dict(sliding_window=8, layer_types=["sliding_attention", "full_attention"])),
    "gpt2": ("GPT2Config", dict(n_embd=128, n_layer=2, n_head=4, n_positions=256)),
    "gpt_bigcode": ("GPTBigCodeConfig", dict(n_embd=128, n_layer=2, n_head=4, n_positions=256)),
    "gpt_bigcode_mha": ("GPTBigCodeConfig", dict(n_embd=128, n_layer=2, n_head=4, n_positions=256, multi_query=False)),
    "falcon": ("FalconConfig", dict(new_decoder_architecture=False, multi_query=True, parallel_attn=True, bias=False, alibi=False)),
    "falcon_grouped": ("FalconConfig", dict(new_decoder_architecture=True, num_kv_heads=2, parallel_attn=True, bias=False, alibi=False)),
    "falcon_mha_bias": ("FalconConfig", dict(new_decoder_architecture=False, multi_query=False, parallel_attn=True, bias=True, alibi=False)),
    "nemotron": ("NemotronConfig", dict()),
    "gpt_neox": ("GPTNeoXConfig", dict()),
    "phi": ("PhiConfig", dict()),
    "opt": ("OPTConfig", dict(ffn_dim=256, word_embed_proj_dim=128)),
    "smollm3": ("SmolLM3Config", dict(pad_token_id=0, no_rope_layer_interval=2)),
    "exaone4": ("Exaone4Config", dict(head_dim=32)),
    "helium": ("HeliumConfig", dict(head_dim=32)),
    "arcee": ("ArceeConfig", dict()),
    "seed_oss": ("SeedOssConfig", dict(head_dim=32)),
    "ministral": ("MinistralConfig", dict(head_dim=32, sliding_window=8,
                                          layer_types=["sliding_attention", "full_attention"])),
    "ernie4_5": ("Ernie4_5Config", dict(head_dim=32)),
    "bloom": ("BloomConfig", dict(n_layer=2, n_head=4)),
    "bloom_6_heads": ("BloomConfig", dict(n_layer=2, n_head=6, hidden_size=192)),
    "gpt_oss": ("GptOssConfig", dict(num_local_experts=4, num_experts_per_tok=2, head_dim=32, sliding_window=8,
                                     layer_types=["sliding_attention", "full_attention"])),
    "hunyuan_v1_dense": ("HunYuanDenseV1Config", dict(head_dim=32)),
    "hunyuan_ntk_alpha": ("HunYuanDenseV1Config", dict(head_dim=32, rope_parameters=dict(rope_type="dynamic", alpha=50.0, rope_theta=10000.0, factor=1.0))),
    "apertus": ("ApertusConfig", dict()),
    "granitemoe": ("GraniteMoeConfig", dict(num_local_experts=4, num_experts_per_tok=2, intermediate_size=64, residual_multiplier=0.5,
                                            embedding_multiplier=3.0, logits_scaling=2.0, attention_multiplier=0.2)),
    "granitemoeshared": ("GraniteMoeSharedConfig", dict(num_local_experts=4, num_experts_per_tok=2, intermediate_size=64,
                                                        shared_intermediate_size=96, residual_multiplier=0.5, logits_scaling=2.0)),
    "olmo": ("OlmoConfig", dict()),
    "olmo3": ("Olmo3Config", dict(sliding_window=8, layer_types=["sliding_attention", "full_attention"])),
    "gptj": ("GPTJConfig", dict(n_embd=128, n_layer=2, n_head=4, n_positions=256, rotary_dim=16)),
    "deepseek_v2": ("DeepseekV2Config", dict(n_routed_experts=4, num_experts_per_tok=2, moe_intermediate_size=64, q_lora_rank=64,
                                             kv_lora_rank=512, qk_nope_head_dim=32, qk_rope_head_dim=64, v_head_dim=32, n_group=1,
                                             topk_group=1, first_k_dense_replace=1, n_shared_experts=1, num_key_value_heads=4)),
    "glm4_moe": ("Glm4MoeConfig", dict(n_routed_experts=4, num_experts_per_tok=2, moe_intermediate_size=64, n_group=1, topk_group=1,
                                       first_k_dense_replace=1, n_shared_experts=1, head_dim=32)),
    "dots1": ("Dots1Config", dict(n_routed_experts=4, num_experts_per_tok=2, moe_intermediate_size=64, n_group=1, topk_group=1,
                                  first_k_dense_replace=1, n_shared_experts=1, head_dim=32)),
    "cwm": ("CwmConfig", dict()),
    "ernie4_5_moe": ("Ernie4_5_MoeConfig", dict(moe_num_experts=4, moe_k=2, moe_intermediate_size=64, head_dim=32, moe_layer_start_index=1,
                                                moe_num_shared_experts=1)),
    "hunyuan_v1_moe": ("HunYuanMoEV1Config", dict(num_experts=4, moe_topk=2, head_dim=32)),
    "deepseek_v3": ("DeepseekV3Config", dict(n_routed_experts=4, num_experts_per_tok=2, moe_intermediate_size=64,
                                             q_lora_rank=64, kv_lora_rank=512, qk_nope_head_dim=32, qk_rope_head_dim=64,
                                             v_head_dim=32, n_group=2, topk_group=1, first_k_dense_replace=1,
                                             n_shared_experts=1, num_key_value_heads=4)),
}


def _logits(llm, ids):
    m = llm.model
    n = len(ids)
    m.alloc_kv((n + 15) // 16 + 1, 16)
    b = ForwardBatch(tokens=torch.tensor(ids, dtype=torch.int32), positions=torch.arange(n, dtype=torch.int32),
                     slot_mapping=torch.arange(n, dtype=torch.int32),
                     block_table=torch.arange((n + 15) // 16 + 1, dtype=torch.int32)[None],
                     kv_lens=torch.tensor([n], dtype=torch.int32), is_decode=False,
                     cu_q=torch.tensor([0, n], dtype=torch.int32), max_q_len=n, max_kv_len=n)
    return m.logits(m.forward_hidden(b)).float()


@pytest.mark.parametrize("name", sorted(ARCHS))
def test_arch_matches_transformers(name, tmp_path):
    cls, extra = ARCHS[name]
    if not hasattr(tr, cls):
        pytest.skip(f"transformers has no {cls}")
    cfg = getattr(tr, cls)(**{**_BASE, **extra})
    cfg._attn_implementation = "eager"
    torch.manual_seed(0)
    hf = tr.AutoModelForCausalLM.from_config(cfg).eval()
    with torch.no_grad():
        for p in hf.parameters():            # default init is tiny; widen so that every branch matters
            if p.ndim >= 2:
                if not bool(p.any()):         # a router the library leaves at zero: every expert would tie
                    p.normal_(0, 0.02)
                p.mul_(3.0)
            elif "norm" in "".join(n for n, q in hf.named_parameters() if q is p):
                p.add_(torch.randn_like(p) * 0.1)
    d = tmp_path / name
    save_hf_checkpoint(cfg.to_dict(), {k: v.detach().to(torch.bfloat16).contiguous() for k, v in hf.state_dict().items()}, d)
    hf = hf.to(torch.bfloat16).float()       # the same rounded weights on both sides
    llm = load_llm(d, "cpu")
    ids = torch.randint(0, 320, (23,), generator=torch.Generator().manual_seed(1)).tolist()
    with torch.no_grad():
        ref = hf(torch.tensor([ids])).logits[0].float()
    mine = _logits(llm, ids)
    cos = torch.nn.functional.cosine_similarity(mine.flatten(), ref.flatten(), dim=0)
    assert cos > 0.995, f"{name}: cos {cos:.4f}"
    agree = (mine.argmax(-1) == ref.argmax(-1)).float().mean()
    assert agree >= 0.85, f"{name}: argmax agreement {agree:.2f}"


GGUF_ARCHS = ["bloom", "llama", "mistral", "qwen2", "qwen3", "gemma", "gemma2", "gemma3_text", "granite", "olmo2", "phi3",
              "stablelm", "stablelm_parallel", "starcoder2", "gpt_neox", "mixtral", "qwen2_moe", "qwen3_moe", "olmoe",
              "deepseek_v3"]


@pytest.mark.parametrize("name", GGUF_ARCHS)
def test_converted_gguf_matches_the_hf_directory(name, tmp_path):
    """HF directory -> GGUF (llama.cpp names, permuted q/k, stacked experts, baked Gemma norms) ->
    loaded again: same logits as the directory it came from."""
    from hartsyinference_b200.assets.converters import hf_to_gguf
    cls, extra = ARCHS[name]
    cfg = getattr(tr, cls)(**{**_BASE, **extra})
    torch.manual_seed(0)
    hf = tr.AutoModelForCausalLM.from_config(cfg)
    with torch.no_grad():
        for p in hf.parameters():
            if p.ndim >= 2:
                p.mul_(3.0)
            else:
                p.add_(torch.randn_like(p) * 0.1)
    d = tmp_path / name
    save_hf_checkpoint(cfg.to_dict(), {k: v.detach().to(torch.bfloat16).contiguous() for k, v in hf.state_dict().items()}, d)
    md = hf_to_gguf(d, tmp_path / f"{name}.gguf")
    assert md["general.architecture"]
    a, b = load_llm(d, "cpu"), load_llm(tmp_path / f"{name}.gguf", "cpu")
    ids = torch.randint(0, 320, (19,), generator=torch.Generator().manual_seed(2)).tolist()
    la, lb = _logits(a, ids), _logits(b, ids)
    cos = torch.nn.functional.cosine_similarity(la.flatten(), lb.flatten(), dim=0)
    assert cos > 0.999, f"{name}: cos {cos:.4f}"
    assert (la.argmax(-1) == lb.argmax(-1)).float().mean() >= 0.9


def test_convert_verb_writes_a_quantised_gguf_with_its_tokenizer(tmp_path):
    import json
    from click.testing import CliRunner
    from hartsyinference_b200.assets.gguf import GgufFile
    from hartsyinference_b200.cli.main import cli
    cfg = tr.Qwen2Config(**_BASE)
    torch.manual_seed(0)
    hf = tr.AutoModelForCausalLM.from_config(cfg)
    d = tmp_path / "q"
    save_hf_checkpoint(cfg.to_dict(), {k: v.detach().to(torch.bfloat16).contiguous() for k, v in hf.state_dict().items()}, d)
    from hartsyinference_b200.assets.tokenizer import _bytes_to_unicode
    b2u = _bytes_to_unicode()
    vocab = {b2u[b]: b for b in range(256)}
    vocab[b2u[ord("h")] + b2u[ord("i")]] = 256
    (d / "tokenizer.json").write_text(json.dumps({
        "model": {"type": "BPE", "vocab": vocab, "merges": [f"{b2u[ord('h')]} {b2u[ord('i')]}"]},
        "added_tokens": [{"id": 300, "content": "<|end|>", "special": True}]}))
    (d / "tokenizer_config.json").write_text(json.dumps({"chat_template": "{{ messages[0]['content'] }}"}))
    r = CliRunner().invoke(cli, ["convert", str(d), str(tmp_path / "q.gguf"), "--quant", "Q8_0"])
    assert r.exit_code == 0, r.output
    f = GgufFile(tmp_path / "q.gguf")
    assert f.info("blk.0.attn_q.weight")[0] == 8 and f.info("blk.0.attn_norm.weight")[0] == 0     # Q8_0 / F32
    assert f.metadata["tokenizer.chat_template"].startswith("{{") and f.metadata["tokenizer.ggml.tokens"][300] == "<|end|>"
    a, b = load_llm(d, "cpu"), load_llm(tmp_path / "q.gguf", "cpu")
    assert b.tokenizer.encode("hi", add_special=False) == a.tokenizer.encode("hi", add_special=False) == [256]
    ids = list(range(5, 20))
    cos = torch.nn.functional.cosine_similarity(_logits(a, ids).flatten(), _logits(b, ids).flatten(), dim=0)
    assert cos > 0.99


def test_internlm2_and_minicpm_map_onto_the_llama_block(tmp_path):
    """No transformers class exists for these two: InternLM 2 is checked by regrouping a llama
    checkpoint into its fused per-kv-group layout, MiniCPM by its scaling rules against Granite's."""
    from hartsyinference_b200.models.llm.config import from_hf_config
    cfg = tr.LlamaConfig(**_BASE)
    torch.manual_seed(0)
    hf = tr.AutoModelForCausalLM.from_config(cfg)
    sd = {k: v.detach().to(torch.bfloat16).contiguous() for k, v in hf.state_dict().items()}
    save_hf_checkpoint(cfg.to_dict(), sd, tmp_path / "llama")
    heads, kvh, d = 4, 2, 32
    ren = {"model.embed_tokens.weight": "model.tok_embeddings.weight", "lm_head.weight": "output.weight",
           "model.norm.weight": "model.norm.weight"}
    out = {ren[k]: v for k, v in sd.items() if k in ren}
    for i in range(2):
        p = f"model.layers.{i}."
        q = sd[p + "self_attn.q_proj.weight"].reshape(kvh, heads // kvh, d, -1)
        k = sd[p + "self_attn.k_proj.weight"].reshape(kvh, 1, d, -1)
        v = sd[p + "self_attn.v_proj.weight"].reshape(kvh, 1, d, -1)
        out[p + "attention.wqkv.weight"] = torch.cat([q, k, v], 1).reshape(-1, q.shape[-1]).contiguous()
        out[p + "attention.wo.weight"] = sd[p + "self_attn.o_proj.weight"]
        out[p + "feed_forward.w1.weight"] = sd[p + "mlp.gate_proj.weight"]
        out[p + "feed_forward.w3.weight"] = sd[p + "mlp.up_proj.weight"]
        out[p + "feed_forward.w2.weight"] = sd[p + "mlp.down_proj.weight"]
        out[p + "attention_norm.weight"] = sd[p + "input_layernorm.weight"]
        out[p + "ffn_norm.weight"] = sd[p + "post_attention_layernorm.weight"]
    save_hf_checkpoint({**cfg.to_dict(), "model_type": "internlm2"}, out, tmp_path / "internlm2")
    ids = list(range(3, 24))
    a, b = _logits(load_llm(tmp_path / "llama", "cpu"), ids), _logits(load_llm(tmp_path / "internlm2", "cpu"), ids)
    assert torch.equal(a, b)

    mc = from_hf_config({**cfg.to_dict(), "model_type": "minicpm", "scale_emb": 12.0, "scale_depth": 1.4, "dim_model_base": 32})
    assert mc.embedding_multiplier == 12.0 and abs(mc.residual_multiplier - 1.4 / 2 ** 0.5) < 1e-9 and mc.logits_scale == 0.25
    save_hf_checkpoint({**cfg.to_dict(), "model_type": "minicpm", "scale_emb": 12.0, "scale_depth": 1.4, "dim_model_base": 32},
                       sd, tmp_path / "minicpm")
    save_hf_checkpoint({**cfg.to_dict(), "model_type": "granite", "embedding_multiplier": 12.0,
                        "residual_multiplier": 1.4 / 2 ** 0.5, "logits_scaling": 4.0, "attention_multiplier": d ** -0.5},
                       sd, tmp_path / "granite")
    c, e = _logits(load_llm(tmp_path / "minicpm", "cpu"), ids), _logits(load_llm(tmp_path / "granite", "cpu"), ids)
    assert torch.allclose(c, e, atol=1e-3)


def test_alibi_decode_step_matches_prefill(tmp_path):
    """BLOOM's attention runs through the gathered-page path: a decode step after a prefill gives
    the logits the one-shot prefill gives for the same position."""
    cfg = tr.BloomConfig(**{**_BASE, "n_layer": 2, "n_head": 4})
    torch.manual_seed(0)
    hf = tr.AutoModelForCausalLM.from_config(cfg).eval()
    save_hf_checkpoint(cfg.to_dict(), {k: v.detach().to(torch.bfloat16).contiguous() for k, v in hf.state_dict().items()},
                       tmp_path / "m")
    llm = load_llm(tmp_path / "m", "cpu")
    ids = torch.randint(0, 320, (19,), generator=torch.Generator().manual_seed(2)).tolist()
    full = _logits(llm, ids)[-1]
    m = llm.model
    _logits(llm, ids[:-1])
    n = len(ids)
    b = ForwardBatch(tokens=torch.tensor(ids[-1:], dtype=torch.int32), positions=torch.tensor([n - 1], dtype=torch.int32),
                     slot_mapping=torch.tensor([n - 1], dtype=torch.int32),
                     block_table=torch.arange((n + 15) // 16 + 1, dtype=torch.int32)[None],
                     kv_lens=torch.tensor([n], dtype=torch.int32), is_decode=True, max_kv_len=n)
    step = m.logits(m.forward_hidden(b)).float()[0]
    assert torch.nn.functional.cosine_similarity(step, full, dim=0) > 0.999
    assert int(step.argmax()) == int(full.argmax())


def test_gpt_oss_mxfp4_expert_blocks_load(tmp_path):
    """Released gpt-oss checkpoints keep the expert matrices as MXFP4 blocks + E8M0 scales, laid out
    [E, out, in / 32, 16]: they load to the same logits as the dequantised matrices stored plainly."""
    from hartsyinference_b200.assets.lowbit import mxfp4_dequantize, mxfp4_quantize
    cfg = tr.GptOssConfig(**{**_BASE, **ARCHS["gpt_oss"][1]})
    torch.manual_seed(0)
    sd = {k: v.detach().to(torch.bfloat16).contiguous() for k, v in tr.AutoModelForCausalLM.from_config(cfg).state_dict().items()}
    plain, packed = dict(sd), dict(sd)
    for k in list(sd):
        if k.endswith(("experts.gate_up_proj", "experts.down_proj")):
            w = sd[k].float().transpose(1, 2).contiguous()                       # [E, out, in]
            e, rows, cols = w.shape
            q, sc = mxfp4_quantize(w.reshape(e * rows, cols))
            plain[k] = mxfp4_dequantize(q, sc).reshape(e, rows, cols).transpose(1, 2).contiguous().to(torch.bfloat16)
            del packed[k]
            packed[k + "_blocks"] = q.reshape(e, rows, cols // 32, 16)
            packed[k + "_scales"] = sc.reshape(e, rows, cols // 32)
    save_hf_checkpoint(cfg.to_dict(), plain, tmp_path / "plain")
    save_hf_checkpoint(cfg.to_dict(), packed, tmp_path / "packed")
    ids = torch.randint(0, 320, (17,), generator=torch.Generator().manual_seed(3)).tolist()
    a = _logits(load_llm(tmp_path / "plain", "cpu"), ids)
    b = _logits(load_llm(tmp_path / "packed", "cpu"), ids)
    assert torch.equal(a, b)


def _mllama(tmp_path):
    cfg = tr.models.mllama.configuration_mllama.MllamaTextConfig(**{**_BASE, "cross_attention_layers": [1], "num_hidden_layers": 3, "pad_token_id": 0,
                                               "rope_parameters": {"rope_type": "default", "rope_theta": 10000.0}})
    cfg._attn_implementation = "eager"
    torch.manual_seed(0)
    hf = tr.MllamaForCausalLM(cfg).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if p.ndim >= 2:
                p.mul_(3.0)
            if n.endswith(("cross_attn_attn_gate", "cross_attn_mlp_gate")):
                p.fill_(0.7)                                     # the gates initialise to zero (identity layer)
    save_hf_checkpoint(cfg.to_dict(), {k: v.detach().to(torch.bfloat16).contiguous() for k, v in hf.state_dict().items()},
                       tmp_path / "m")
    return hf.to(torch.bfloat16).float(), load_llm(tmp_path / "m", "cpu")


def test_mllama_text_only_skips_cross_layers(tmp_path):
    hf, llm = _mllama(tmp_path)
    assert llm.config.cross_layers == (1,) and llm.model.layers[1].cross is not None
    ids = torch.randint(0, 320, (21,), generator=torch.Generator().manual_seed(1)).tolist()
    with torch.no_grad():
        ref = hf(torch.tensor([ids])).logits[0].float()
    mine = _logits(llm, ids)
    assert torch.nn.functional.cosine_similarity(mine.flatten(), ref.flatten(), dim=0) > 0.995


def test_mllama_cross_attention_over_vision_states(tmp_path):
    hf, llm = _mllama(tmp_path)
    ids = torch.randint(0, 320, (21,), generator=torch.Generator().manual_seed(1)).tolist()
    states = torch.randn(1, 12, 128, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16)
    rows = torch.ones(1, 1, 21, 1)
    rows[:, :, :4] = 0                                           # the first text rows precede the image
    with torch.no_grad():
        ref = hf(torch.tensor([ids]), cross_attention_states=states.float(), full_text_row_masked_out_mask=rows).logits[0].float()
        plain = hf(torch.tensor([ids])).logits[0].float()
    m, n = llm.model, len(ids)
    m.alloc_kv((n + 15) // 16 + 1, 16)
    b = ForwardBatch(tokens=torch.tensor(ids, dtype=torch.int32), positions=torch.arange(n, dtype=torch.int32),
                     slot_mapping=torch.arange(n, dtype=torch.int32),
                     block_table=torch.arange((n + 15) // 16 + 1, dtype=torch.int32)[None],
                     kv_lens=torch.tensor([n], dtype=torch.int32), is_decode=False,
                     cu_q=torch.tensor([0, n], dtype=torch.int32), max_q_len=n, max_kv_len=n,
                     cross_states=states[0], cross_row_mask=rows[0, 0, :, 0])
    mine = m.logits(m.forward_hidden(b)).float()
    assert torch.nn.functional.cosine_similarity(ref.flatten(), plain.flatten(), dim=0) < 0.98      # the image matters
    assert torch.nn.functional.cosine_similarity(mine.flatten(), ref.flatten(), dim=0) > 0.995


def test_mllama_engine_batches_requests_with_and_without_images(tmp_path):
    """Through the engine: a request with vision states and a text-only one decode in the same
    batch, and each produces what it produces alone; the image request follows transformers' greedy
    continuation."""
    from hartsyinference_b200.engine.llm_engine import LLMEngine, SamplingParams
    hf, llm = _mllama(tmp_path)
    g = torch.Generator().manual_seed(5)
    a = torch.randint(0, 320, (9,), generator=g).tolist()
    b = torch.randint(0, 320, (13,), generator=g).tolist()
    states = (torch.randn(10, 128, generator=g) * 2).to(torch.bfloat16)
    sp = SamplingParams(greedy=True, max_tokens=5)

    def run(jobs):
        eng = LLMEngine(llm.model, num_pages=32, page_size=16, max_batch=4, prefill_chunk=64, max_model_len=64)
        rids = [eng.add_request(ids, sp, cross_states=st) for ids, st in jobs]
        eng.run_until_done()
        return [eng.requests[r].output for r in rids]

    both = run([(a, states), (b, None)])
    assert both[0] == run([(a, states)])[0]
    assert both[1] == run([(b, None)])[0]
    assert both[0] != run([(a, None)])[0]
    with torch.no_grad():
        ref = hf.generate(torch.tensor([a]), cross_attention_states=states[None].float(), max_new_tokens=5, do_sample=False,
                          pad_token_id=0)[0, len(a):].tolist()
    assert both[0][:len(ref)] == ref
