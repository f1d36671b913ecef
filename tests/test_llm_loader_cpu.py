"""Synthetic checkpoints written to disk load through both containers and agree with each other."""
import json

import torch

from hartsyinference_b200.assets import gguf as G
from hartsyinference_b200.engine import LLMEngine, SamplingParams
from hartsyinference_b200.models.llm.loader import load_llm, save_hf_checkpoint


def _synthetic(seed=0, qkv_bias=True, tie=True, heads=4, kvh=2, d=32):
    g = torch.Generator().manual_seed(seed)
    h, L, ffn, vocab = heads * d, 2, 256, 300
    cfg = {"model_type": "qwen2", "vocab_size": vocab, "hidden_size": h, "num_hidden_layers": L,
           "num_attention_heads": heads, "num_key_value_heads": kvh, "intermediate_size": ffn,
           "rms_norm_eps": 1e-6, "rope_theta": 1e6, "tie_word_embeddings": tie, "max_position_embeddings": 512,
           "eos_token_id": 299, "bos_token_id": 298}
    t = {}
    rn = lambda *s: (torch.randn(*s, generator=g) * 0.05).to(torch.bfloat16)
    t["model.embed_tokens.weight"] = rn(vocab, h)
    t["model.norm.weight"] = torch.ones(h, dtype=torch.bfloat16)
    if not tie:
        t["lm_head.weight"] = rn(vocab, h)
    for i in range(L):
        p = f"model.layers.{i}."
        t[p + "self_attn.q_proj.weight"] = rn(heads * d, h); t[p + "self_attn.k_proj.weight"] = rn(kvh * d, h)
        t[p + "self_attn.v_proj.weight"] = rn(kvh * d, h); t[p + "self_attn.o_proj.weight"] = rn(h, heads * d)
        if qkv_bias:
            t[p + "self_attn.q_proj.bias"] = rn(heads * d); t[p + "self_attn.k_proj.bias"] = rn(kvh * d)
            t[p + "self_attn.v_proj.bias"] = rn(kvh * d)
        t[p + "mlp.gate_proj.weight"] = rn(ffn, h); t[p + "mlp.up_proj.weight"] = rn(ffn, h)
        t[p + "mlp.down_proj.weight"] = rn(h, ffn)
        t[p + "input_layernorm.weight"] = torch.ones(h, dtype=torch.bfloat16)
        t[p + "post_attention_layernorm.weight"] = torch.ones(h, dtype=torch.bfloat16)
    return cfg, t


def _to_gguf(cfg, tensors, path, quant=None):
    inv_layer = {"input_layernorm.weight": "attn_norm.weight", "self_attn.q_proj.weight": "attn_q.weight",
                 "self_attn.q_proj.bias": "attn_q.bias", "self_attn.k_proj.weight": "attn_k.weight",
                 "self_attn.k_proj.bias": "attn_k.bias", "self_attn.v_proj.weight": "attn_v.weight",
                 "self_attn.v_proj.bias": "attn_v.bias", "self_attn.o_proj.weight": "attn_output.weight",
                 "post_attention_layernorm.weight": "ffn_norm.weight", "mlp.gate_proj.weight": "ffn_gate.weight",
                 "mlp.up_proj.weight": "ffn_up.weight", "mlp.down_proj.weight": "ffn_down.weight"}
    out = {}
    for k, v in tensors.items():
        if k == "model.embed_tokens.weight":
            out["token_embd.weight"] = v
        elif k == "model.norm.weight":
            out["output_norm.weight"] = v
        elif k == "lm_head.weight":
            out["output.weight"] = v
        else:
            _, _, idx, rest = k.split(".", 3)
            out[f"blk.{idx}.{inv_layer[rest]}"] = v
    md = {"general.architecture": "qwen2", "qwen2.block_count": cfg["num_hidden_layers"],
          "qwen2.embedding_length": cfg["hidden_size"], "qwen2.attention.head_count": cfg["num_attention_heads"],
          "qwen2.attention.head_count_kv": cfg["num_key_value_heads"], "qwen2.feed_forward_length": cfg["intermediate_size"],
          "qwen2.attention.layer_norm_rms_epsilon": 1e-6, "qwen2.rope.freq_base": 1e6, "qwen2.context_length": 512,
          "qwen2.vocab_size": cfg["vocab_size"], "tokenizer.ggml.bos_token_id": 298, "tokenizer.ggml.eos_token_id": 299}
    G.write_gguf(path, md, out, quant=quant)


def test_hf_dir_and_gguf_give_the_same_generation(tmp_path):
    cfg, t = _synthetic()
    save_hf_checkpoint(cfg, t, tmp_path / "hf")
    _to_gguf(cfg, t, tmp_path / "m.gguf")
    a = load_llm(tmp_path / "hf", "cpu")
    b = load_llm(tmp_path / "m.gguf", "cpu")
    assert a.config.num_kv_heads == b.config.num_kv_heads == 2 and a.config.qkv_bias and b.config.tie_embeddings
    p = SamplingParams(greedy=True, ignore_eos=True, max_tokens=6)
    prompt = a.tokenizer.encode("hello")
    outs = []
    for lm in (a, b):
        e = LLMEngine(lm.model, num_pages=16, page_size=16, max_batch=2, prefill_chunk=64, max_model_len=128)
        outs.append(e.generate([prompt], p)[0])
    assert outs[0] == outs[1]


def test_quantised_gguf_stays_close(tmp_path):
    cfg, t = _synthetic(seed=3, qkv_bias=False, tie=False)
    _to_gguf(cfg, t, tmp_path / "f.gguf")
    _to_gguf(cfg, t, tmp_path / "q.gguf", quant=G.GGML_TYPES["Q8_0"])
    a, b = load_llm(tmp_path / "f.gguf", "cpu"), load_llm(tmp_path / "q.gguf", "cpu")
    wa, wb = a.model.layers[0].qkv.weight.float(), b.model.layers[0].qkv.weight.float()
    assert ((wa - wb).norm() / wa.norm()).item() < 0.02
    assert not a.config.tie_embeddings


def test_gguf_blocks_kept_resident_give_the_same_tokens(tmp_path):
    from hartsyinference_b200 import config, ops
    cfg, t = _synthetic(3, qkv_bias=False)
    _to_gguf(cfg, t, tmp_path / "q.gguf", quant=G.GGML_TYPES["Q8_0"])
    a = load_llm(tmp_path / "q.gguf", "cpu")
    config.set_override("gguf_resident", True)
    try:
        b = load_llm(tmp_path / "q.gguf", "cpu")
    finally:
        config.set_override("gguf_resident", None)
    lw = b.model.layers[0]
    assert isinstance(lw.qkv, ops.GgufWeight) and isinstance(lw.down, ops.GgufWeight)
    assert lw.qkv.out_features == a.model.layers[0].qkv.out_features
    p = SamplingParams(greedy=True, max_tokens=8, ignore_eos=True)
    ea = LLMEngine(a.model, num_pages=32, page_size=16, max_batch=2, prefill_chunk=64, max_model_len=128)
    eb = LLMEngine(b.model, num_pages=32, page_size=16, max_batch=2, prefill_chunk=64, max_model_len=128)
    prompt = [[3, 9, 27, 81, 5]]
    assert ea.generate(prompt, p) == eb.generate(prompt, p)
    assert b.model.weight_bytes() < a.model.weight_bytes()
