"""Load a decoder LLM from a Hugging Face directory (``config.json`` + safetensors shards) or from a
GGUF file, together with its tokenizer and chat template.

Counterpart of ``GgufLanguageModel.Load`` (GGUF -> config -> tokenizer -> chat template ->
transformer; src/HartsyInference.LLM/Generation/GgufLanguageModel.cs:206) and of the per-architecture
GGUF key mappers (src/HartsyInference.ModelAssets/Gguf/KeyMappers/). The reference loads text LLMs
from GGUF only; safetensors directories are accepted here as well.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Callable, Optional

import torch

from ... import log
from ...assets.chat_template import ChatTemplate
from ...assets.gguf import GgufFile
from ...assets.safetensors import ShardedCheckpoint
from ...assets.tokenizer import ByteTokenizer, Tokenizer
from ...exceptions import UnsupportedModelError
from ...parallel.comm import Comm
from .config import TransformerConfig, from_gguf_metadata, from_hf_config
from .transformer import DecoderModel

# GGUF tensor name -> Hugging Face name (llama-family layout shared by qwen2/3, mistral, gemma, ...)
_GGUF_LAYER = {
    "attn_norm.weight": "input_layernorm.weight",
    "attn_q.weight": "self_attn.q_proj.weight", "attn_q.bias": "self_attn.q_proj.bias",
    "attn_k.weight": "self_attn.k_proj.weight", "attn_k.bias": "self_attn.k_proj.bias",
    "attn_v.weight": "self_attn.v_proj.weight", "attn_v.bias": "self_attn.v_proj.bias",
    "attn_output.weight": "self_attn.o_proj.weight",
    "attn_q_norm.weight": "self_attn.q_norm.weight", "attn_k_norm.weight": "self_attn.k_norm.weight",
    "ffn_norm.weight": "post_attention_layernorm.weight",
    "ffn_gate.weight": "mlp.gate_proj.weight", "ffn_up.weight": "mlp.up_proj.weight",
    "ffn_down.weight": "mlp.down_proj.weight",
    "post_attention_norm.weight": "post_attention_layernorm.weight",
    "post_ffw_norm.weight": "post_feedforward_layernorm.weight",
    # LayerNorm / linear biases (StableLM, StarCoder 2, GPT-NeoX)
    "attn_norm.bias": "input_layernorm.bias", "ffn_norm.bias": "post_attention_layernorm.bias",
    "attn_output.bias": "self_attn.o_proj.bias", "ffn_up.bias": "mlp.up_proj.bias", "ffn_down.bias": "mlp.down_proj.bias",
    "ffn_gate.bias": "mlp.gate_proj.bias",
    # fused projections (Phi-3, GPT-NeoX): sliced by ``standard_names``
    "attn_qkv.weight": "self_attn.qkv_proj.weight", "attn_qkv.bias": "self_attn.qkv_proj.bias",
    # mixture of experts: stacked [experts, out, in] tensors
    "ffn_gate_inp.weight": "mlp.gate.weight", "exp_probs_b.bias": "mlp.gate.e_score_correction_bias",
    "ffn_down_exps.weight": "mlp.experts.down_proj",
    "ffn_gate_shexp.weight": "mlp.shared_experts.gate_proj.weight", "ffn_up_shexp.weight": "mlp.shared_experts.up_proj.weight",
    "ffn_down_shexp.weight": "mlp.shared_experts.down_proj.weight", "ffn_gate_inp_shexp.weight": "mlp.shared_expert_gate.weight",
    # multi-head latent attention
    "attn_q_a.weight": "self_attn.q_a_proj.weight", "attn_q_a_norm.weight": "self_attn.q_a_layernorm.weight",
    "attn_q_b.weight": "self_attn.q_b_proj.weight", "attn_kv_a_mqa.weight": "self_attn.kv_a_proj_with_mqa.weight",
    "attn_kv_a_norm.weight": "self_attn.kv_a_layernorm.weight", "attn_kv_b.weight": "self_attn.kv_b_proj.weight",
}
_GGUF_TOP = {"token_embd.weight": "model.embed_tokens.weight", "output_norm.weight": "model.norm.weight",
             "output_norm.bias": "model.norm.bias", "output.weight": "lm_head.weight",
             "token_embd_norm.weight": "model.embed_norm.weight", "token_embd_norm.bias": "model.embed_norm.bias"}


def gguf_name_to_hf(name: str) -> Optional[str]:
    if name in _GGUF_TOP:
        return _GGUF_TOP[name]
    if name.startswith("blk."):
        _, idx, rest = name.split(".", 2)
        hf = _GGUF_LAYER.get(rest)
        if hf:
            return f"model.layers.{idx}.{hf}"
    return None


@dataclass
class LoadedLLM:
    model: DecoderModel
    tokenizer: Tokenizer
    chat_template: ChatTemplate
    config: TransformerConfig
    source: str
    vlm: Optional[object] = None      # LlavaModel when the checkpoint carries a vision tower


def _gemma_sandwich_fix(cfg: TransformerConfig, get: Callable[[str], Optional[torch.Tensor]]):
    """GGUF Gemma-2/3 files name the pre-FFN norm ``ffn_norm`` and the post-attention norm
    ``post_attention_norm``; the model expects HF names."""
    if not cfg.post_norms:
        return get

    def wrapped(name: str):
        if name.endswith("pre_feedforward_layernorm.weight"):
            return get(name.replace("pre_feedforward_layernorm", "__ffn_norm__"))
        return get(name)
    return wrapped


def load_llm(path: str | Path, device: str | torch.device = "cuda", comm: Optional[Comm] = None,
             fp8: Optional[bool] = None) -> LoadedLLM:
    if str(path).startswith("synthetic:"):
        return _load_synthetic(str(path)[len("synthetic:"):], device, comm, fp8)
    p = Path(path)
    if p.is_file() and p.suffix == ".gguf":
        return _load_gguf(p, device, comm, fp8)
    if p.is_dir() and (p / "config.json").exists():
        return _load_hf(p, device, comm, fp8)
    if p.is_dir():
        ggufs = sorted(p.glob("*.gguf"))
        if ggufs:
            return _load_gguf(ggufs[0], device, comm, fp8)
    raise UnsupportedModelError(f"{path}: neither a .gguf file nor a directory with config.json")


def _load_synthetic(spec: str, device, comm: Optional[Comm], fp8: Optional[bool]) -> LoadedLLM:
    """``synthetic:<preset>[:layers=N]``: the named architecture with random-init weights (seed 0)
    and a byte tokenizer padded to the vocabulary size. For benchmarks and smoke tests of the
    serving stack where no checkpoint is at hand; prompts are best passed as token ids."""
    from ...assets.tokenizer import ByteTokenizer
    from .config import PRESETS
    name, *mods = spec.split(":")
    if name not in PRESETS:
        raise UnsupportedModelError(f"synthetic:{name}: unknown preset (known: {sorted(PRESETS)})")
    cfg = PRESETS[name]
    for m in mods:
        k, _, v = m.partition("=")
        if k == "layers":
            from dataclasses import replace
            cfg = replace(cfg, num_layers=int(v))
        else:
            raise UnsupportedModelError(f"synthetic:{spec}: unknown modifier {k!r}")
    model = DecoderModel(cfg, device, comm=comm, fp8=_want_fp8(fp8, device), dp_attention=_want_dp_attention(cfg, comm))
    model.random_init(seed=0)
    return LoadedLLM(model, ByteTokenizer(vocab_size=cfg.vocab_size), ChatTemplate.for_arch(cfg.arch), cfg, f"synthetic:{spec}")


def _want_dp_attention(cfg, comm) -> bool:
    """Latent-attention models on more than one rank also keep the attention weights of all heads, for
    the data-parallel attention layout of decode steps (parallel/dp_attention.py)."""
    from ... import config
    return cfg.mla is not None and comm is not None and comm.world > 1 and bool(config.get("dp_attention"))


def _want_fp8(fp8: Optional[bool], device) -> bool:
    from ... import config
    if fp8 is not None:
        return fp8
    return bool(config.get("fp8_linears")) and torch.device(device).type == "cuda"


def standard_names(get: Callable[[str], Optional[torch.Tensor]], raw: dict) -> Callable[[str], Optional[torch.Tensor]]:
    """Present an architecture's own tensor names and fused tensors under the llama-style names the
    decoder loads (``model.layers.N.self_attn.q_proj.weight`` ...): Phi-3 / GLM fused projections are
    sliced, GLM-4 / StarCoder 2 / GPT-NeoX names are translated, GPT-NeoX's per-head interleaved
    query_key_value is regrouped."""
    mt = raw.get("model_type", "llama")
    heads = raw.get("num_attention_heads") or raw.get("n_head") or 1
    hidden = raw.get("hidden_size", 0)
    d = raw.get("head_dim") or (hidden // heads if heads else 0)
    kvh = raw.get("num_key_value_heads") or heads

    def fused_rows(name: str, fused: str, part: str, sizes: dict[str, tuple[int, int]]):
        t = get(name.replace(part, fused))
        if t is None:
            return None
        a, b = sizes[part]
        return t[a:b]

    if mt == "phi3" or mt in ("glm", "glm4"):
        qs, ks = heads * d, kvh * d
        qkv = {"q_proj": (0, qs), "k_proj": (qs, qs + ks), "v_proj": (qs + ks, qs + 2 * ks)}
        ffn = raw.get("intermediate_size", 0)
        gu = {"gate_proj": (0, ffn), "up_proj": (ffn, 2 * ffn)}
        glm4 = {"post_attention_layernorm": "post_self_attn_layernorm", "pre_feedforward_layernorm": "post_attention_layernorm",
                "post_feedforward_layernorm": "post_mlp_layernorm"}

        def g(name: str):
            if mt == "glm4":
                for std, own in glm4.items():
                    if "." + std + "." in name:
                        return get(name.replace(std, own))
            t = get(name)
            if t is not None:
                return t
            for part in qkv:
                if "self_attn." + part + "." in name:
                    return fused_rows(name, "qkv_proj", part, qkv)
            for part in gu:
                if "mlp." + part + "." in name:
                    return fused_rows(name, "gate_up_proj", part, gu)
            return None
        return g
    if mt == "gpt_bigcode":
        # GPT-2 names with ordinary [out, in] Linear weights; the fused projection is [hidden | k | v] with one shared
        # key / value head when multi_query, else per head [q | k | v]
        h = raw.get("n_embd", hidden)
        ren = (("model.embed_tokens", "transformer.wte"), ("model.embed_positions", "transformer.wpe"),
               ("model.norm", "transformer.ln_f"), ("model.layers", "transformer.h"), ("input_layernorm", "ln_1"),
               ("post_attention_layernorm", "ln_2"), ("self_attn.o_proj", "attn.c_proj"), ("mlp.up_proj", "mlp.c_fc"),
               ("mlp.down_proj", "mlp.c_proj"))
        mq = bool(raw.get("multi_query", True))
        hd = h // heads

        def g(name: str):
            for i, part in enumerate(("q_proj", "k_proj", "v_proj")):
                if "self_attn." + part + "." in name:
                    t = get(name.replace("model.layers", "transformer.h").replace("self_attn." + part, "attn.c_attn"))
                    if t is None:
                        return None
                    if mq:
                        return (t[:h] if i == 0 else t[h + (i - 1) * hd:h + i * hd]).contiguous()
                    return t.reshape(heads, 3, hd, *t.shape[1:])[:, i].reshape(h, *t.shape[1:]).contiguous()
            own = name
            for std, o in ren:
                own = own.replace(std, o)
            return get(own)
        return g
    if mt == "gpt2":
        h = raw.get("n_embd", hidden)
        ren = (("model.embed_tokens", "transformer.wte"), ("model.embed_positions", "transformer.wpe"),
               ("model.norm", "transformer.ln_f"), ("model.layers", "transformer.h"), ("input_layernorm", "ln_1"),
               ("post_attention_layernorm", "ln_2"), ("self_attn.o_proj", "attn.c_proj"), ("mlp.up_proj", "mlp.c_fc"),
               ("mlp.down_proj", "mlp.c_proj"))

        def g(name: str):
            for i, part in enumerate(("q_proj", "k_proj", "v_proj")):
                if "self_attn." + part + "." in name:
                    t = get(name.replace("model.layers", "transformer.h").replace("self_attn." + part, "attn.c_attn"))
                    if t is None:
                        return None
                    t = t.t() if t.dim() == 2 else t          # Conv1D keeps [in, out]
                    return t[i * h:(i + 1) * h].contiguous()
            own = name
            for std, o in ren:
                own = own.replace(std, o)
            t = get(own)
            if t is not None and t.dim() == 2 and (".attn.c_proj." in own or ".mlp.c_" in own):
                t = t.t().contiguous()
            return t
        return g
    if mt == "internlm2":
        groups = heads // kvh
        ren = (("model.embed_tokens", "model.tok_embeddings"), ("lm_head", "output"), ("input_layernorm", "attention_norm"),
               ("post_attention_layernorm", "ffn_norm"), ("self_attn.o_proj", "attention.wo"),
               ("mlp.gate_proj", "feed_forward.w1"), ("mlp.up_proj", "feed_forward.w3"), ("mlp.down_proj", "feed_forward.w2"))

        def g(name: str):
            for part in ("q_proj", "k_proj", "v_proj"):
                if "self_attn." + part + "." in name:
                    t = get(name.replace("self_attn." + part, "attention.wqkv"))
                    if t is None:
                        return None
                    # rows are [kv head][its q heads..., k, v][d]
                    t = t.reshape(kvh, groups + 2, d, *t.shape[1:])
                    sel = t[:, :groups] if part == "q_proj" else t[:, groups + (0 if part == "k_proj" else 1)][:, None]
                    return sel.reshape(-1, *t.shape[3:]).contiguous()
            for std, own in ren:
                name = name.replace(std, own)
            return get(name)
        return g
    if mt == "olmo":
        # OLMo 1 normalises with a LayerNorm that has no parameters: present a weight of ones
        def g(name: str):
            t = get(name)
            if t is None and name.endswith(("layernorm.weight", "model.norm.weight")):
                return torch.ones(hidden, dtype=torch.bfloat16)
            return t
        return g
    if mt in ("hunyuan_v1_dense", "hunyuan_v1_moe"):
        def g(name: str):
            return get(name.replace("self_attn.q_norm", "self_attn.query_layernorm").replace("self_attn.k_norm", "self_attn.key_layernorm"))
        return g
    if mt in ("granitemoe", "granitemoeshared"):
        sf = int(raw.get("shared_intermediate_size") or 0)

        def shared(name: str):          # shared_mlp keeps gate | up in one input_linear
            base = name[: name.index("mlp.shared_experts.")] + "shared_mlp."
            if name.endswith("down_proj.weight"):
                return get(base + "output_linear.weight")
            t = get(base + "input_linear.weight")
            return None if t is None else (t[:sf] if name.endswith("gate_proj.weight") else t[sf:])
        ren = (("mlp.gate.weight", "block_sparse_moe.router.layer.weight"), ("mlp.experts.gate_up_proj", "block_sparse_moe.input_linear.weight"),
               ("mlp.experts.down_proj", "block_sparse_moe.output_linear.weight"))

        def g(name: str):
            if "mlp.shared_experts." in name:
                return shared(name) if sf else None
            for std, own in ren:
                if name.endswith(std):
                    return get(name[: -len(std)] + own)
            return get(name)
        return g
    if mt == "apertus":
        def g(name: str):
            return get(name.replace("input_layernorm", "attention_layernorm").replace("post_attention_layernorm", "feedforward_layernorm"))
        return g
    if mt == "opt":
        layer = (("input_layernorm", "self_attn_layer_norm"), ("post_attention_layernorm", "final_layer_norm"),
                 ("self_attn.o_proj", "self_attn.out_proj"), ("mlp.up_proj", "fc1"), ("mlp.down_proj", "fc2"))

        def g(name: str):
            if name.startswith("model.layers."):
                for std, own in layer:
                    name = name.replace(std, own)
                return get("model.decoder." + name[len("model."):])
            if name.startswith("model.norm."):
                return get("model.decoder.final_layer_norm." + name[len("model.norm."):])
            if name.startswith("model.embed_"):
                return get("model.decoder." + name[len("model."):])
            return get(name)
        return g
    if mt == "gptj":
        ren = (("model.embed_tokens", "transformer.wte"), ("model.norm", "transformer.ln_f"), ("model.layers", "transformer.h"),
               ("input_layernorm", "ln_1"), ("self_attn.o_proj", "attn.out_proj"), ("self_attn.", "attn."),
               ("mlp.up_proj", "mlp.fc_in"), ("mlp.down_proj", "mlp.fc_out"))

        def g(name: str):
            for std, own in ren:
                name = name.replace(std, own)
            return get(name)
        return g
    if mt == "phi":
        ren = (("model.norm", "model.final_layernorm"), ("self_attn.o_proj", "self_attn.dense"), ("mlp.up_proj", "mlp.fc1"),
               ("mlp.down_proj", "mlp.fc2"))

        def g(name: str):
            for std, own in ren:
                name = name.replace(std, own)
            return get(name)
        return g
    if mt == "starcoder2":
        return lambda name: get(name.replace("mlp.up_proj", "mlp.c_fc").replace("mlp.down_proj", "mlp.c_proj"))
    if mt == "bloom":
        ren = (("model.embed_tokens", "transformer.word_embeddings"), ("model.embed_norm", "transformer.word_embeddings_layernorm"),
               ("model.norm", "transformer.ln_f"), ("model.layers", "transformer.h"), ("self_attn.o_proj", "self_attention.dense"),
               ("mlp.up_proj", "mlp.dense_h_to_4h"), ("mlp.down_proj", "mlp.dense_4h_to_h"))

        def g(name: str):
            for i, part in enumerate(("q_proj", "k_proj", "v_proj")):
                if "self_attn." + part + "." in name:
                    t = get(name.replace("model.layers", "transformer.h").replace("self_attn." + part, "self_attention.query_key_value"))
                    if t is None:
                        return None
                    return t.reshape(heads, 3, d, *t.shape[1:])[:, i].reshape(heads * d, *t.shape[1:])   # rows are [head][q | k | v][d]
            for std, own in ren:
                name = name.replace(std, own)
            return get(name)
        return g
    if mt == "falcon":
        new = bool(raw.get("new_decoder_architecture", False))
        two_norms = new and (raw.get("num_ln_in_parallel_attn") or 2) == 2
        ren = (("model.embed_tokens", "transformer.word_embeddings"), ("model.norm", "transformer.ln_f"), ("model.layers", "transformer.h"),
               ("self_attn.o_proj", "self_attention.dense"), ("mlp.up_proj", "mlp.dense_h_to_4h"), ("mlp.down_proj", "mlp.dense_4h_to_h")) + \
              ((("input_layernorm", "ln_attn"), ("post_attention_layernorm", "ln_mlp")) if two_norms else ())
        kvf = (raw.get("num_kv_heads") or heads) if new else (1 if raw.get("multi_query", True) else heads)
        groups = heads // kvf

        def g(name: str):
            for i, part in enumerate(("q_proj", "k_proj", "v_proj")):
                if "self_attn." + part + "." in name:
                    t = get(name.replace("model.layers", "transformer.h").replace("self_attn." + part, "self_attention.query_key_value"))
                    if t is None:
                        return None
                    if new:                                  # rows are [kv head][its q heads..., k, v][d]
                        t = t.reshape(kvf, groups + 2, d, *t.shape[1:])
                        sel = t[:, :groups] if i == 0 else t[:, groups + i - 1][:, None]
                        return sel.reshape(-1, *t.shape[3:]).contiguous()
                    if kvf == 1:                             # multi-query: [all q heads | k | v]
                        return (t[:heads * d] if i == 0 else t[heads * d + (i - 1) * d:heads * d + i * d]).contiguous()
                    return t.reshape(heads, 3, d, *t.shape[1:])[:, i].reshape(heads * d, *t.shape[1:]).contiguous()
            for std, own in ren:
                name = name.replace(std, own)
            return get(name)
        return g
    if mt == "gpt_neox":
        ren = (("model.embed_tokens", "gpt_neox.embed_in"), ("model.norm", "gpt_neox.final_layer_norm"),
               ("lm_head", "embed_out"), ("model.layers", "gpt_neox.layers"), ("self_attn.o_proj", "attention.dense"),
               ("mlp.up_proj", "mlp.dense_h_to_4h"), ("mlp.down_proj", "mlp.dense_4h_to_h"))

        def g(name: str):
            for i, part in enumerate(("q_proj", "k_proj", "v_proj")):
                if "self_attn." + part + "." in name:
                    own = name.replace("model.layers", "gpt_neox.layers").replace("self_attn." + part, "attention.query_key_value")
                    t = get(own)
                    if t is None:
                        return None
                    # rows are [head][q | k | v][d]
                    return t.reshape(heads, 3, d, *t.shape[1:])[:, i].reshape(heads * d, *t.shape[1:])
            for std, own in ren:
                name = name.replace(std, own)
            return get(name)
        return g
    return get


def _llava_names(ck) -> tuple[Callable, Callable]:
    """Two checkpoint layouts exist for LLaVA: ``language_model.model.* / language_model.lm_head /
    vision_tower.* / multi_modal_projector.*`` and the later ``model.language_model.* /
    model.vision_tower.* / model.multi_modal_projector.* / lm_head``. Returns (decoder get, tower get)
    that take the plain decoder names and the first layout's tower names."""
    new = ck.get("model.language_model.embed_tokens.weight") is not None
    flat = ck.get("model.embed_tokens.weight") is not None        # decoder names unprefixed (first Qwen-VL releases)

    def lm(name: str):
        if flat:
            return ck.get(name)
        if new:
            return ck.get("model.language_model." + name[len("model."):]) if name.startswith("model.") else ck.get(name)
        return ck.get("language_model." + name)

    def tower(name: str):
        return ck.get(("model." if new else "") + name)

    return lm, tower


def _load_hf(p: Path, device, comm, fp8) -> LoadedLLM:
    from ...assets.lowbit import dequantizing_get
    raw = json.loads((p / "config.json").read_text())
    ck = ShardedCheckpoint(p)
    vlm = None
    ck_get = dequantizing_get(ck.get)          # fp8 block-scaled / NVFP4 / MXFP4 / NF4 linears read as bf16
    if "vision_config" in raw and "text_config" in raw:
        from ..encoders.clip_vision import clip_vision_from_hf
        from ..vlm.llava import LlavaModel
        text = dict(raw["text_config"])
        text.setdefault("model_type", "llama")
        cfg = from_hf_config(text)
        lm_get, tower_get = _llava_names(ck)
        if raw.get("model_type") in ("idefics3", "smolvlm"):
            # decoder tensors sit under model.text_model.*
            lm_get = lambda name: ck.get("model.text_model." + name[len("model."):]) if name.startswith("model.") else ck.get(name)
        model = DecoderModel(cfg, device, comm=comm, fp8=_want_fp8(fp8, device), dp_attention=_want_dp_attention(cfg, comm))
        model.load_state_dict(lm_get)
        if raw.get("model_type") in ("idefics3", "smolvlm"):
            from ..vlm.idefics3 import Idefics3Model, idefics3_vision_from_hf
            edge = None
            pp = p / "preprocessor_config.json"
            if pp.exists():
                edge = (json.loads(pp.read_text()).get("size") or {}).get("longest_edge")
            vlm = Idefics3Model(model, idefics3_vision_from_hf(raw["vision_config"]), int(raw.get("image_token_id", 128257)),
                                int(raw.get("scale_factor", 2)), get=ck.get, longest_edge=edge)
        elif raw.get("model_type") in ("qwen2_5_vl", "qwen2_vl", "qwen3_vl"):
            from ..vlm.qwen_vl import Qwen3VisionConfig, QwenVisionConfig, QwenVlModel
            vcfg = (Qwen3VisionConfig if raw["model_type"] == "qwen3_vl" else QwenVisionConfig).from_hf(raw["vision_config"])
            vlm = QwenVlModel(model, vcfg, ck.get, int(raw.get("image_token_id", 151655)),
                              prefix="model.visual." if ck.get("model.visual.patch_embed.proj.weight") is not None else "visual.",
                              vision_start_id=raw.get("vision_start_token_id"), vision_end_id=raw.get("vision_end_token_id"))
        elif raw.get("model_type") == "mllama":
            from ..vlm.mllama import MllamaModel, MllamaVisionConfig
            new = ck.get("model.language_model.embed_tokens.weight") is not None
            vlm = MllamaModel(model, MllamaVisionConfig.from_hf(raw["vision_config"]), ck.get, int(raw.get("image_token_index", 128256)),
                              tower_prefix="model.vision_model." if new else "vision_model.",
                              projector_prefix="model.multi_modal_projector." if new else "multi_modal_projector.")
        elif raw.get("model_type") == "llava_next" or raw.get("image_grid_pinpoints"):
            from ..vlm.llava_next import DEFAULT_PINPOINTS, LlavaNextModel
            vlm = LlavaNextModel(model, clip_vision_from_hf(raw["vision_config"]), int(raw.get("image_token_index", 32000)),
                                 get=tower_get, feature_layer=int(raw.get("vision_feature_layer", -2)),
                                 pinpoints=[tuple(p) for p in raw.get("image_grid_pinpoints") or DEFAULT_PINPOINTS])
        else:
            vlm = LlavaModel(model, clip_vision_from_hf(raw["vision_config"]), int(raw.get("image_token_index", 32000)),
                             get=tower_get, feature_layer=int(raw.get("vision_feature_layer", -2)))
    else:
        cfg = from_hf_config(raw)
        model = DecoderModel(cfg, device, comm=comm, fp8=_want_fp8(fp8, device), dp_attention=_want_dp_attention(cfg, comm))
        model.load_state_dict(standard_names(ck_get, raw))
    tok: Tokenizer
    if (p / "tokenizer.json").exists():
        tok = Tokenizer.from_hf_json(p / "tokenizer.json")
    else:
        tok = ByteTokenizer(vocab_size=cfg.vocab_size)
    tpl_src, bos, eos = None, "", ""
    tc = p / "tokenizer_config.json"
    if tc.exists():
        d = json.loads(tc.read_text())
        tpl_src = d.get("chat_template")
        bos = d.get("bos_token") if isinstance(d.get("bos_token"), str) else ""
        eos = d.get("eos_token") if isinstance(d.get("eos_token"), str) else ""
    tpl = ChatTemplate(tpl_src, bos or "", eos or "") if tpl_src else ChatTemplate.for_arch(cfg.arch)
    if vlm is not None and hasattr(vlm, "bind_tokenizer"):
        specials = getattr(tok, "special_tokens", None) or {}
        vlm.bind_tokenizer(specials.get, tok.encode("\n", add_special=False))
    log.info(f"[Load] {p.name}: {cfg.arch} {cfg.num_layers}L hidden {cfg.hidden_size} "
             f"({model.weight_bytes() / 2**30:.2f} GiB on {device})")
    return LoadedLLM(model, tok, tpl, cfg, str(p), vlm)


def _load_gguf(p: Path, device, comm, fp8) -> LoadedLLM:
    f = GgufFile(p)
    cfg = from_gguf_metadata(f.metadata)
    hf_to_gguf = {}
    for name in f.keys():
        hf = gguf_name_to_hf(name)
        if hf:
            hf_to_gguf[hf] = name
    if cfg.post_norms:   # Gemma 2/3 (and OLMo 2, which has no ffn_norm): ffn_norm is the pre-FFN norm
        for i in range(cfg.num_layers):
            a = f"model.layers.{i}.post_attention_layernorm.weight"
            g = f"blk.{i}.ffn_norm.weight"
            if g in f:
                hf_to_gguf[f"model.layers.{i}.pre_feedforward_layernorm.weight"] = g
            g2 = f"blk.{i}.post_attention_norm.weight"
            if g2 in f:
                hf_to_gguf[a] = g2

    def get_plain(name: str) -> Optional[torch.Tensor]:
        g = hf_to_gguf.get(name)
        if g is not None:
            return f.get(g, torch.bfloat16)
        if name.endswith("mlp.experts.gate_up_proj"):          # gate and up expert stacks side by side
            blk = "blk." + name.split(".")[2]
            if blk + ".ffn_gate_exps.weight" in f:
                return torch.cat([f.get(blk + ".ffn_gate_exps.weight", torch.bfloat16),
                                  f.get(blk + ".ffn_up_exps.weight", torch.bfloat16)], 1)
        return None

    arch = f.metadata.get("general.architecture", "llama")
    fused = {"phi3": "phi3", "gptneox": "phi3", "bloom": "phi3"}.get(arch)
    if fused:
        # both keep q|k|v (and Phi-3 gate|up in ffn_up) as one tensor: present them under the split names
        raw = {"model_type": "phi3", "num_attention_heads": cfg.num_heads, "num_key_value_heads": cfg.num_kv_heads,
               "hidden_size": cfg.hidden_size, "head_dim": cfg.head_dim, "intermediate_size": cfg.ffn_size}
        if arch == "phi3":
            for i in range(cfg.num_layers):
                hf_to_gguf[f"model.layers.{i}.mlp.gate_up_proj.weight"] = hf_to_gguf.pop(f"model.layers.{i}.mlp.up_proj.weight")
        get = standard_names(get_plain, raw)
    else:
        get = get_plain

    from ... import config as _config
    resident = bool(_config.get("gguf_resident")) and (comm is None or comm.world == 1)
    model = DecoderModel(cfg, device, comm=comm, fp8=_want_fp8(fp8, device) and not resident,
                         dp_attention=_want_dp_attention(cfg, comm))
    model.load_state_dict(get)
    if resident:
        kept = _keep_gguf_blocks(model, f, hf_to_gguf)
        log.decision("Load", f"{kept} linear(s) kept as GGUF blocks on {model.device}")
    tok = Tokenizer.from_gguf_metadata(f.metadata) if "tokenizer.ggml.tokens" in f.metadata else ByteTokenizer(vocab_size=cfg.vocab_size)
    src = f.metadata.get("tokenizer.chat_template")
    tokens = f.metadata.get("tokenizer.ggml.tokens") or []
    bos_id, eos_id = f.metadata.get("tokenizer.ggml.bos_token_id"), f.metadata.get("tokenizer.ggml.eos_token_id")
    bos = tokens[bos_id] if isinstance(bos_id, int) and bos_id < len(tokens) else ""
    eos = tokens[eos_id] if isinstance(eos_id, int) and eos_id < len(tokens) else ""
    tpl = ChatTemplate(src, bos, eos) if src else ChatTemplate.for_arch(cfg.arch)
    log.info(f"[Load] {p.name}: GGUF v{f.version} {cfg.arch} {cfg.num_layers}L hidden {cfg.hidden_size}")
    return LoadedLLM(model, tok, tpl, cfg, str(p))


def _keep_gguf_blocks(model: DecoderModel, f: GgufFile, hf_to_gguf: dict[str, str]) -> int:
    """Replace the dense linears of a single-rank model by :class:`ops.GgufWeight` views of the
    file's own Q8_0 / Q4_K blocks (fused q/k/v and gate/up rows are concatenated block rows).
    A linear whose tensors have mixed or unsupported types keeps its dequantised weight."""
    from ... import ops

    def blocks_of(hf_names: list[str]):
        raws, typ, k = [], None, None
        for hn in hf_names:
            g = hf_to_gguf.get(hn)
            if g is None:
                return None
            t, shape = f.info(g)
            if len(shape) != 2 or not ops.GgufWeight.supported(t, shape[1]) or (typ is not None and (t, shape[1]) != (typ, k)):
                return None
            typ, k = t, shape[1]
            raws.append(ops.GgufWeight.from_raw(f.raw(g).clone(), t, shape[0], shape[1]).blocks)
        return ops.GgufWeight(torch.cat(raws).to(model.device).contiguous(), typ, k)

    kept = 0
    for i, lw in enumerate(model.layers):
        p = f"model.layers.{model.layer0 + i}."
        plan = {"qkv": [p + f"self_attn.{n}_proj.weight" for n in ("q", "k", "v")], "o": [p + "self_attn.o_proj.weight"],
                "gate_up": [p + "mlp.gate_proj.weight", p + "mlp.up_proj.weight"], "down": [p + "mlp.down_proj.weight"]}
        for attr, names in plan.items():
            cur = getattr(lw, attr)
            if cur is None or cur.bias is not None:
                continue
            gw = blocks_of(names)
            if gw is not None and gw.out_features == cur.out_features and gw.k == cur.in_features:
                setattr(lw, attr, gw)
                kept += 1
    return kept


def save_hf_checkpoint(model_cfg: dict, tensors: dict[str, torch.Tensor], out_dir: str | Path) -> None:
    """Write ``config.json`` + ``model.safetensors`` (used to build synthetic checkpoints)."""
    from ...assets.safetensors import save_file
    d = Path(out_dir)
    d.mkdir(parents=True, exist_ok=True)
    (d / "config.json").write_text(json.dumps(model_cfg, indent=1))
    save_file(tensors, d / "model.safetensors", {"format": "pt"})
