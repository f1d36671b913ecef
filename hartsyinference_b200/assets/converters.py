"""Checkpoint converters: a Hugging Face decoder directory -> one GGUF file (llama.cpp's metadata
keys and tensor names), with optional block quantisation of the 2-D weights.

What the conversion does beyond renaming: llama-family q / k rows are permuted to the interleaved
rotary layout those GGUF files use, Gemma's ``w - 1`` norm weights get their 1 added, per-expert
tensors are stacked into ``[experts, out, in]`` blocks, fused projections (Phi-3, GPT-NeoX) are
written the way llama.cpp keeps them, and the tokenizer (vocabulary, merges, special ids, chat
template) is embedded.

Reference: src/HartsyInference.ModelAssets/CheckpointConverters/.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Optional

import torch

from . import gguf as G
from .safetensors import ShardedCheckpoint

# Hugging Face model_type -> GGUF architecture name
ARCH = {"llama": "llama", "mistral": "llama", "mixtral": "llama", "qwen2": "qwen2", "qwen3": "qwen3", "gemma": "gemma",
        "gemma2": "gemma2", "gemma3_text": "gemma3", "gemma3": "gemma3", "phi3": "phi3", "olmo2": "olmo2",
        "granite": "granite", "stablelm": "stablelm", "starcoder2": "starcoder2", "gpt_neox": "gptneox",
        "qwen2_moe": "qwen2moe", "qwen3_moe": "qwen3moe", "olmoe": "olmoe", "deepseek_v3": "deepseek2",
        "deepseek_v2": "deepseek2", "bloom": "bloom"}

# architectures whose GGUF files rotate interleaved pairs: q / k rows are permuted on the way in
_PERMUTE_QK = {"llama", "granite"}

_LAYER = {
    "input_layernorm": "attn_norm", "self_attn.q_proj": "attn_q", "self_attn.k_proj": "attn_k", "self_attn.v_proj": "attn_v",
    "self_attn.o_proj": "attn_output", "self_attn.q_norm": "attn_q_norm", "self_attn.k_norm": "attn_k_norm",
    "post_attention_layernorm": "ffn_norm", "mlp.gate_proj": "ffn_gate", "mlp.up_proj": "ffn_up", "mlp.down_proj": "ffn_down",
    "pre_feedforward_layernorm": "ffn_norm", "post_feedforward_layernorm": "post_ffw_norm",
    "self_attn.qkv_proj": "attn_qkv", "mlp.gate_up_proj": "ffn_up", "mlp.c_fc": "ffn_up", "mlp.c_proj": "ffn_down",
    "attention.query_key_value": "attn_qkv", "attention.dense": "attn_output", "mlp.dense_h_to_4h": "ffn_up",
    "mlp.dense_4h_to_h": "ffn_down", "self_attention.query_key_value": "attn_qkv", "self_attention.dense": "attn_output",
    "mlp.gate": "ffn_gate_inp", "block_sparse_moe.gate": "ffn_gate_inp", "mlp.shared_expert_gate": "ffn_gate_inp_shexp",
    "mlp.shared_expert.gate_proj": "ffn_gate_shexp", "mlp.shared_expert.up_proj": "ffn_up_shexp",
    "mlp.shared_expert.down_proj": "ffn_down_shexp", "mlp.shared_experts.gate_proj": "ffn_gate_shexp",
    "mlp.shared_experts.up_proj": "ffn_up_shexp", "mlp.shared_experts.down_proj": "ffn_down_shexp",
    "self_attn.q_a_proj": "attn_q_a", "self_attn.q_a_layernorm": "attn_q_a_norm", "self_attn.q_b_proj": "attn_q_b",
    "self_attn.kv_a_proj_with_mqa": "attn_kv_a_mqa", "self_attn.kv_a_layernorm": "attn_kv_a_norm",
    "self_attn.kv_b_proj": "attn_kv_b",
}
_TOP = {"model.embed_tokens": "token_embd", "model.norm": "output_norm", "lm_head": "output",
        "gpt_neox.embed_in": "token_embd", "gpt_neox.final_layer_norm": "output_norm", "embed_out": "output",
        "transformer.word_embeddings": "token_embd", "transformer.word_embeddings_layernorm": "token_embd_norm",
        "transformer.ln_f": "output_norm"}


def permute_qk(w: torch.Tensor, heads: int) -> torch.Tensor:
    """Split-half rotary row order -> interleaved-pair order, per head (rows [h][2][d/2] -> [h][d/2][2])."""
    rows = w.shape[0]
    return w.reshape(heads, 2, rows // heads // 2, *w.shape[1:]).transpose(1, 2).reshape(w.shape)


def _metadata(raw: dict, arch: str, vocab: int) -> dict:
    heads = raw["num_attention_heads"]
    hidden = raw["hidden_size"]
    d = raw.get("head_dim") or hidden // heads
    rp = raw.get("rope_parameters") or raw.get("rope_scaling") or {}
    if "full_attention" in rp:
        rp = rp["full_attention"] or {}
    eps = next((raw[k] for k in ("rms_norm_eps", "layer_norm_eps", "norm_epsilon", "norm_eps") if raw.get(k) is not None), 1e-5)
    md = {"general.architecture": arch, "general.name": raw.get("_name_or_path") or arch,
          f"{arch}.block_count": raw["num_hidden_layers"], f"{arch}.embedding_length": hidden,
          f"{arch}.attention.head_count": heads, f"{arch}.attention.head_count_kv": raw.get("num_key_value_heads") or heads,
          f"{arch}.feed_forward_length": raw.get("intermediate_size") or 4 * hidden,
          f"{arch}.attention.layer_norm_rms_epsilon": float(eps), f"{arch}.attention.layer_norm_epsilon": float(eps),
          f"{arch}.rope.freq_base": float(raw.get("rope_theta") or rp.get("rope_theta") or 10000.0),
          f"{arch}.context_length": raw.get("max_position_embeddings", 8192), f"{arch}.vocab_size": vocab,
          f"{arch}.attention.key_length": d, f"{arch}.attention.value_length": d}
    prf = raw.get("partial_rotary_factor") or rp.get("partial_rotary_factor") or raw.get("rotary_pct")
    if prf and float(prf) < 1.0:
        md[f"{arch}.rope.dimension_count"] = int(d * float(prf))
    if rp.get("rope_type", rp.get("type")) == "linear":
        md[f"{arch}.rope.scaling.type"] = "linear"
        md[f"{arch}.rope.scaling.factor"] = float(rp.get("factor", 1.0))
    for key, name in (("sliding_window", "attention.sliding_window"), ("final_logit_softcapping", "final_logit_softcapping"),
                      ("attn_logit_softcapping", "attn_logit_softcapping")):
        if raw.get(key):
            md[f"{arch}.{name}"] = raw[key]
    if raw.get("query_pre_attn_scalar"):
        md[f"{arch}.attention.scale"] = float(raw["query_pre_attn_scalar"]) ** -0.5
    if arch == "granite":
        md.update({"granite.attention.scale": float(raw.get("attention_multiplier", 0.0)),
                   "granite.residual_scale": float(raw.get("residual_multiplier", 1.0)),
                   "granite.embedding_scale": float(raw.get("embedding_multiplier", 1.0)),
                   "granite.logit_scale": float(raw.get("logits_scaling", 1.0))})
    if arch == "gptneox":
        md["gptneox.use_parallel_residual"] = bool(raw.get("use_parallel_residual", True))
    if arch == "stablelm":
        md["stablelm.use_parallel_residual"] = bool(raw.get("use_parallel_residual", False))
    n_exp = raw.get("num_experts") or raw.get("num_local_experts") or raw.get("n_routed_experts")
    if n_exp:
        md.update({f"{arch}.expert_count": n_exp, f"{arch}.expert_used_count": raw.get("num_experts_per_tok", 2),
                   f"{arch}.expert_feed_forward_length": raw.get("moe_intermediate_size") or raw.get("intermediate_size"),
                   f"{arch}.expert_weights_norm": bool(raw.get("norm_topk_prob", raw.get("model_type") == "mixtral"))})
        if raw.get("shared_expert_intermediate_size"):
            md[f"{arch}.expert_shared_feed_forward_length"] = raw["shared_expert_intermediate_size"]
            md[f"{arch}.expert_shared_count"] = 1
    if arch == "deepseek2":
        md.update({"deepseek2.attention.q_lora_rank": raw.get("q_lora_rank") or 0,
                   "deepseek2.attention.kv_lora_rank": raw["kv_lora_rank"],
                   "deepseek2.attention.key_length": raw["qk_nope_head_dim"] + raw["qk_rope_head_dim"],
                   "deepseek2.attention.value_length": raw["v_head_dim"],
                   "deepseek2.rope.dimension_count": raw["qk_rope_head_dim"],
                   "deepseek2.expert_shared_count": raw.get("n_shared_experts") or 0,
                   "deepseek2.expert_shared_feed_forward_length": raw.get("moe_intermediate_size") or 0,
                   "deepseek2.expert_weights_scale": float(raw.get("routed_scaling_factor", 1.0)),
                   "deepseek2.expert_gating_func": 2 if raw.get("scoring_func", "sigmoid" if raw.get("model_type") == "deepseek_v3" else "softmax") == "sigmoid" else 1,
                   "deepseek2.expert_group_count": raw.get("n_group") or 1,
                   "deepseek2.expert_group_used_count": raw.get("topk_group") or 1,
                   "deepseek2.leading_dense_block_count": raw.get("first_k_dense_replace", 0)})
    bos, eos = raw.get("bos_token_id"), raw.get("eos_token_id")
    if isinstance(bos, int):
        md["tokenizer.ggml.bos_token_id"] = bos
    if eos is not None:
        md["tokenizer.ggml.eos_token_id"] = int(eos[0] if isinstance(eos, (list, tuple)) else eos)
    return md


def _tokenizer_metadata(src: Path, md: dict, vocab: int) -> None:
    """Embed a byte-level BPE ``tokenizer.json`` (vocabulary, merges, token types, chat template)."""
    tj = src / "tokenizer.json"
    if not tj.exists():
        return
    data = json.loads(tj.read_text(encoding="utf-8"))
    model = data.get("model") or {}
    if model.get("type") != "BPE":
        return
    toks = [""] * vocab
    types = [1] * vocab
    for t, i in (model.get("vocab") or {}).items():
        if i < vocab:
            toks[i] = t
    for a in data.get("added_tokens") or []:
        if a["id"] < vocab:
            toks[a["id"]] = a["content"]
            types[a["id"]] = 3 if a.get("special") else 4
    md["tokenizer.ggml.model"] = "gpt2"
    md["tokenizer.ggml.tokens"] = toks
    md["tokenizer.ggml.token_type"] = types
    md["tokenizer.ggml.merges"] = [m if isinstance(m, str) else " ".join(m) for m in model.get("merges") or []]
    tc = src / "tokenizer_config.json"
    if tc.exists():
        tpl = json.loads(tc.read_text(encoding="utf-8")).get("chat_template")
        if isinstance(tpl, str):
            md["tokenizer.chat_template"] = tpl


def hf_to_gguf(src_dir, dst, quant: Optional[str] = None) -> dict:
    """Convert the decoder checkpoint in ``src_dir`` to the GGUF file ``dst``. ``quant`` names a ggml
    block type (``Q8_0``, ``Q4_0``, ``Q4_K``) for the 2-D weights; norms, biases and stacked expert
    tensors stay F32. Returns the metadata that was written."""
    src = Path(src_dir)
    raw = json.loads((src / "config.json").read_text())
    mt = raw.get("model_type", "llama")
    if mt not in ARCH:
        raise ValueError(f"no GGUF mapping for model_type '{mt}'")
    arch = ARCH[mt]
    ck = ShardedCheckpoint(src)
    if arch == "bloom":                                      # BLOOM names its sizes n_head / n_layer
        raw = {**raw, "num_attention_heads": raw["n_head"], "num_hidden_layers": raw["n_layer"],
               "rms_norm_eps": raw.get("layer_norm_epsilon", 1e-5), "max_position_embeddings": raw.get("seq_length", 2048),
               "intermediate_size": 4 * raw["hidden_size"]}
    heads = raw["num_attention_heads"]
    if arch in ("gptneox", "bloom"):
        raw = {**raw, "num_key_value_heads": heads}          # always multi-head
    kvh = raw.get("num_key_value_heads") or heads
    hidden = raw["hidden_size"]
    d = raw.get("head_dim") or hidden // heads
    gemma = arch.startswith("gemma")
    out: dict[str, torch.Tensor] = {}
    experts: dict[tuple[str, str], dict[int, torch.Tensor]] = {}
    vocab = raw["vocab_size"]
    for name in ck.keys():
        t = ck.get(name)
        stem, _, kind = name.rpartition(".")
        if kind not in ("weight", "bias"):
            stem, kind = name, ""                # stacked expert tensors and correction biases have no suffix
        if stem in _TOP:
            if gemma and "norm" in stem:
                t = t.float() + 1.0
            out[f"{_TOP[stem]}.{kind}"] = t
            continue
        parts = stem.split(".")
        if arch == "bloom" and "h" in parts:
            parts[parts.index("h")] = "layers"
        if "layers" not in parts:
            continue
        li = parts.index("layers")
        idx, rest = parts[li + 1], ".".join(parts[li + 2:])
        if name.endswith("e_score_correction_bias"):
            out[f"blk.{idx}.exp_probs_b.bias"] = t
            continue
        if rest in ("mlp.experts.gate_up_proj", "mlp.experts.down_proj"):      # already stacked [E, out, in]
            if rest.endswith("gate_up_proj"):
                f = t.shape[1] // 2
                out[f"blk.{idx}.ffn_gate_exps.weight"], out[f"blk.{idx}.ffn_up_exps.weight"] = t[:, :f], t[:, f:]
            else:
                out[f"blk.{idx}.ffn_down_exps.weight"] = t
            continue
        if ".experts." in "." + rest + ".":                                     # per-expert tensors: stack later
            seg = rest.split(".")
            e = int(seg[seg.index("experts") + 1])
            which = {"gate_proj": "ffn_gate_exps", "w1": "ffn_gate_exps", "up_proj": "ffn_up_exps", "w3": "ffn_up_exps",
                     "down_proj": "ffn_down_exps", "w2": "ffn_down_exps"}[seg[-1]]
            experts.setdefault((idx, which), {})[e] = t
            continue
        g = _LAYER.get(rest)
        if g is None:
            continue
        if gemma and ("norm" in rest):
            t = t.float() + 1.0
        if arch in _PERMUTE_QK and rest in ("self_attn.q_proj", "self_attn.k_proj"):
            t = permute_qk(t, heads if rest.endswith("q_proj") else kvh)
        if rest in ("attention.query_key_value", "self_attention.query_key_value"):           # [head][q | k | v][d] rows -> all q, all k, all v
            t = t.reshape(heads, 3, d, *t.shape[1:]).transpose(0, 1).reshape(t.shape)
        if arch in ("gemma2", "gemma3") and rest == "post_attention_layernorm":
            g = "post_attention_norm"
        if arch == "olmo2" and rest == "post_attention_layernorm":
            g = "post_attention_norm"
        out[f"blk.{idx}.{g}.{kind}"] = t
    for (idx, which), per in experts.items():
        out[f"blk.{idx}.{which}.weight"] = torch.stack([per[e] for e in sorted(per)])
    md = _metadata(raw, arch, vocab)
    if "output.weight" in out:
        md["__has_output_weight__"] = True
    _tokenizer_metadata(src, md, vocab)
    q = None
    if quant:
        typ = G.GGML_TYPES[quant]
        q = {k: typ for k, v in out.items() if v.dim() == 2 and k.endswith(".weight") and "norm" not in k
             and k != "token_embd.weight" and "ffn_gate_inp" not in k}
    G.write_gguf(dst, md, {k: v.float() for k, v in out.items()}, quant=q)
    return md


# ============================================================================================
# Flux transformer: original (Black Forest Labs / ComfyUI) names <-> diffusers names
# ============================================================================================
_FLUX_TOP = {"time_in.in_layer": "time_text_embed.timestep_embedder.linear_1",
             "time_in.out_layer": "time_text_embed.timestep_embedder.linear_2",
             "vector_in.in_layer": "time_text_embed.text_embedder.linear_1",
             "vector_in.out_layer": "time_text_embed.text_embedder.linear_2",
             "guidance_in.in_layer": "time_text_embed.guidance_embedder.linear_1",
             "guidance_in.out_layer": "time_text_embed.guidance_embedder.linear_2",
             "txt_in": "context_embedder", "img_in": "x_embedder", "final_layer.linear": "proj_out"}
_FLUX_DOUBLE = {"img_mod.lin": "norm1.linear", "txt_mod.lin": "norm1_context.linear",
                "img_attn.proj": "attn.to_out.0", "txt_attn.proj": "attn.to_add_out",
                "img_mlp.0": "ff.net.0.proj", "img_mlp.2": "ff.net.2",
                "txt_mlp.0": "ff_context.net.0.proj", "txt_mlp.2": "ff_context.net.2"}
_FLUX_DOUBLE_NORMS = {"img_attn.norm.query_norm.scale": "attn.norm_q.weight", "img_attn.norm.key_norm.scale": "attn.norm_k.weight",
                      "txt_attn.norm.query_norm.scale": "attn.norm_added_q.weight",
                      "txt_attn.norm.key_norm.scale": "attn.norm_added_k.weight"}
_FLUX_SINGLE = {"modulation.lin": "norm.linear", "linear2": "proj_out"}
_FLUX_SINGLE_NORMS = {"norm.query_norm.scale": "attn.norm_q.weight", "norm.key_norm.scale": "attn.norm_k.weight"}
_FLUX_PREFIXES = ("model.diffusion_model.", "diffusion_model.", "transformer.")


def is_flux_original(keys) -> bool:
    return any(k.endswith("double_blocks.0.img_attn.qkv.weight") for k in keys)


def _swap_halves(t: torch.Tensor) -> torch.Tensor:
    """[shift; scale] rows <-> [scale; shift] rows (the two layouts order the AdaLN output differently)."""
    a, b = t.chunk(2, 0)
    return torch.cat([b, a], 0)


def flux_original_to_diffusers(tensors: dict[str, torch.Tensor], hidden: Optional[int] = None) -> dict[str, torch.Tensor]:
    """Rename (and split the fused projections of) an original-layout Flux transformer state dict.
    ``hidden`` is inferred from ``img_in.weight`` when omitted."""
    src = {}
    for k, v in tensors.items():
        for pre in _FLUX_PREFIXES:
            if k.startswith(pre):
                k = k[len(pre):]
                break
        src[k] = v
    H = hidden or src["img_in.weight"].shape[0]
    out: dict[str, torch.Tensor] = {}
    for k, v in src.items():
        stem, _, kind = k.rpartition(".")
        if stem in _FLUX_TOP:
            out[f"{_FLUX_TOP[stem]}.{kind}"] = v
        elif stem == "final_layer.adaLN_modulation.1":
            out[f"norm_out.linear.{kind}"] = _swap_halves(v)
        elif k.startswith("double_blocks."):
            _, i, rest = k.split(".", 2)
            p = f"transformer_blocks.{i}."
            rstem, _, rkind = rest.rpartition(".")
            if rest in _FLUX_DOUBLE_NORMS:
                out[p + _FLUX_DOUBLE_NORMS[rest]] = v
            elif rstem in _FLUX_DOUBLE:
                out[f"{p}{_FLUX_DOUBLE[rstem]}.{rkind}"] = v
            elif rstem in ("img_attn.qkv", "txt_attn.qkv"):
                names = ("attn.to_q", "attn.to_k", "attn.to_v") if rstem.startswith("img") else \
                        ("attn.add_q_proj", "attn.add_k_proj", "attn.add_v_proj")
                for n, part in zip(names, v.chunk(3, 0)):
                    out[f"{p}{n}.{rkind}"] = part
        elif k.startswith("single_blocks."):
            _, i, rest = k.split(".", 2)
            p = f"single_transformer_blocks.{i}."
            rstem, _, rkind = rest.rpartition(".")
            if rest in _FLUX_SINGLE_NORMS:
                out[p + _FLUX_SINGLE_NORMS[rest]] = v
            elif rstem in _FLUX_SINGLE:
                out[f"{p}{_FLUX_SINGLE[rstem]}.{rkind}"] = v
            elif rstem == "linear1":
                q, kk, vv, mlp = v.split([H, H, H, v.shape[0] - 3 * H], 0)
                for n, part in (("attn.to_q", q), ("attn.to_k", kk), ("attn.to_v", vv), ("proj_mlp", mlp)):
                    out[f"{p}{n}.{rkind}"] = part
    return out


def flux_diffusers_to_original(tensors: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    """The inverse: fuse q / k / v (and the single blocks' MLP input) and restore the original names."""
    inv_top = {v: k for k, v in _FLUX_TOP.items()}
    inv_double = {v: k for k, v in _FLUX_DOUBLE.items()}
    inv_dn = {v: k for k, v in _FLUX_DOUBLE_NORMS.items()}
    inv_single = {v: k for k, v in _FLUX_SINGLE.items()}
    inv_sn = {v: k for k, v in _FLUX_SINGLE_NORMS.items()}
    out: dict[str, torch.Tensor] = {}
    fuse: dict[str, dict[str, torch.Tensor]] = {}
    for k, v in tensors.items():
        stem, _, kind = k.rpartition(".")
        if stem in inv_top:
            out[f"{inv_top[stem]}.{kind}"] = v
        elif stem == "norm_out.linear":
            out[f"final_layer.adaLN_modulation.1.{kind}"] = _swap_halves(v)
        elif k.startswith("transformer_blocks."):
            _, i, rest = k.split(".", 2)
            p = f"double_blocks.{i}."
            rstem, _, rkind = rest.rpartition(".")
            if rest in inv_dn:
                out[p + inv_dn[rest]] = v
            elif rstem in inv_double:
                out[f"{p}{inv_double[rstem]}.{rkind}"] = v
            elif rstem in ("attn.to_q", "attn.to_k", "attn.to_v"):
                fuse.setdefault(f"{p}img_attn.qkv.{rkind}", {})[rstem[-1]] = v
            elif rstem in ("attn.add_q_proj", "attn.add_k_proj", "attn.add_v_proj"):
                fuse.setdefault(f"{p}txt_attn.qkv.{rkind}", {})[rstem[9]] = v
        elif k.startswith("single_transformer_blocks."):
            _, i, rest = k.split(".", 2)
            p = f"single_blocks.{i}."
            rstem, _, rkind = rest.rpartition(".")
            if rest in inv_sn:
                out[p + inv_sn[rest]] = v
            elif rstem in inv_single:
                out[f"{p}{inv_single[rstem]}.{rkind}"] = v
            elif rstem in ("attn.to_q", "attn.to_k", "attn.to_v", "proj_mlp"):
                fuse.setdefault(f"{p}linear1.{rkind}", {})["m" if rstem == "proj_mlp" else rstem[-1]] = v
    for name, parts in fuse.items():
        out[name] = torch.cat([parts[c] for c in ("q", "k", "v", "m") if c in parts], 0)
    return out
