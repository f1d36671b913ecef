"""Decoder configuration: one record drives every supported decoder architecture.

Plays the role of the reference's ``TransformerConfig`` (+ ``MoeConfig`` / ``MlaConfig``;
src/HartsyInference.LLM/Transformer/TransformerConfig.cs:66-140) and of ``GgufConfigFactory``
(src/HartsyInference.LLM/Transformer/GgufConfigFactory.cs), which maps GGUF metadata of ~30
architectures onto that record. Here both GGUF metadata and Hugging Face ``config.json`` map to
the same dataclass.
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace
from typing import Any, Optional


@dataclass(frozen=True)
class MoeConfig:
    num_experts: int = 0
    top_k: int = 0
    expert_ffn: int = 0
    num_shared_experts: int = 0
    shared_ffn: int = 0
    scoring: str = "softmax"            # softmax | sigmoid
    norm_topk_prob: bool = False
    routed_scaling_factor: float = 1.0
    n_group: int = 1                    # DeepSeek-V3 group-limited routing
    topk_group: int = 1
    use_correction_bias: bool = False
    first_dense_layers: int = 0         # leading layers that keep a dense FFN
    shared_gate: bool = False           # shared expert gated by sigmoid(x . w)


@dataclass(frozen=True)
class MlaConfig:
    q_lora_rank: int = 0
    kv_lora_rank: int = 0
    qk_nope_head_dim: int = 0
    qk_rope_head_dim: int = 0
    v_head_dim: int = 0
    attn_scale: float = 0.0             # > 0 overrides 1/sqrt(nope + rope) (YaRN mscale folded in)


@dataclass(frozen=True)
class RopeScaling:
    kind: str = "none"                  # none | linear | llama3 | yarn
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position: int = 8192
    beta_fast: float = 32.0
    beta_slow: float = 1.0
    attn_factor: float = 1.0
    truncate: bool = True               # YaRN: round the correction range to whole dimensions (gpt-oss does not)


@dataclass(frozen=True)
class TransformerConfig:
    arch: str = "llama"
    vocab_size: int = 32000
    hidden_size: int = 4096
    num_layers: int = 32
    num_heads: int = 32
    num_kv_heads: int = 32
    head_dim: int = 128
    ffn_size: int = 11008
    rms_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_dim: int = 0                   # 0 = head_dim (partial rotary otherwise)
    rope_style: int = 0                 # 0 split-half (HF/NeoX), 1 interleaved (GPT-J / GGUF "norm")
    rope_scaling: RopeScaling = field(default_factory=RopeScaling)
    max_position: int = 131072
    tie_embeddings: bool = False
    qkv_bias: bool = False
    o_bias: bool = False
    ffn_bias: bool = False
    qk_norm: bool = False               # per-head RMSNorm on q and k (Qwen3, OLMo2-style)
    activation: str = "silu"            # silu | gelu_tanh
    gated_ffn: bool = True
    norm_plus_one: bool = False         # Gemma (1 + w)
    embed_scale: float = 1.0            # Gemma sqrt(hidden)
    logit_softcap: float = 0.0
    attn_softcap: float = 0.0
    sliding_window: int = 0
    sliding_window_pattern: int = 0     # every n-th layer is global (0 = all layers use the window)
    post_norms: bool = False            # Gemma2/3 sandwich norms
    attn_scale: float = 0.0             # 0 = 1/sqrt(head_dim)
    residual_multiplier: float = 1.0    # Granite
    embedding_multiplier: float = 1.0
    logits_scale: float = 1.0
    pre_norm: bool = True               # False: norms only after the blocks (OLMo 2)
    qk_norm_full: bool = False          # q/k RMSNorm over the whole projection instead of per head (OLMo 2, OLMoE)
    rope_local_theta: float = 0.0       # rotary base of the sliding-window layers when it differs (Gemma 3)
    layer_types: tuple = ()             # explicit per-layer "sliding_attention" / "full_attention"
    norm_type: str = "rms"              # rms | layernorm
    norm_bias: bool = False
    parallel_residual: bool = False     # x + attn(n1(x)) + ffn(n2(x)) (GPT-NeoX, Cohere)
    shared_parallel_norm: bool = False  # the parallel branches share one norm (Cohere)
    use_rope: bool = True               # False: learned absolute positions instead (GPT-2)
    learned_positions: bool = False
    nope_global: bool = False           # full-attention layers carry no rotary embedding (Cohere 2)
    lm_head_bias: bool = False          # the output projection has a bias (Phi-1 / Phi-2)
    mrope_section: tuple = ()           # rotary frequency pairs driven by the time / row / column position (Qwen-VL)
    mrope_interleaved: bool = False     # sections interleaved over the frequency pairs (t h w t h w ...) instead of chunked (Qwen3-VL)
    cross_layers: tuple = ()            # indices of cross-attention layers reading vision states (Mllama)
    qk_norm_after_rope: bool = False    # per-head q/k RMSNorm applied after the rotary embedding (HunYuan)
    attn_sinks: bool = False            # one learned sink logit per head in the attention softmax (gpt-oss)
    alibi: bool = False                 # attention scores get slope[h] * key position; no rotary embedding (BLOOM)
    embed_norm: bool = False            # LayerNorm directly after the token embedding (BLOOM)
    rope_layers: tuple = ()             # per layer: 1 = rotary embedding, 0 = none (SmolLM 3)
    learned_position_offset: int = 0    # rows skipped at the start of the learned position table (OPT: 2)
    moe: Optional[MoeConfig] = None
    mla: Optional[MlaConfig] = None
    bos_token_id: int = 1
    eos_token_ids: tuple = (2,)

    @property
    def rotary_dim(self) -> int:
        return self.rope_dim or self.head_dim

    @property
    def q_size(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_kv_heads * self.head_dim

    def layer_is_moe(self, layer: int) -> bool:
        return self.moe is not None and self.moe.num_experts > 0 and layer >= self.moe.first_dense_layers

    @property
    def general_path(self) -> bool:
        """Architectures whose block structure is outside the fused decode path: they run the same
        kernels through an unfused layer loop."""
        return (not self.pre_norm or self.qk_norm_full or self.norm_type != "rms" or self.parallel_residual
                or not self.use_rope or self.nope_global or bool(self.rope_layers) or self.alibi or self.embed_norm or self.attn_sinks or self.qk_norm_after_rope or bool(self.cross_layers) or bool(self.mrope_section)
                or self.o_bias or self.ffn_bias or not self.gated_ffn or self.activation not in ("silu", "gelu_tanh"))

    @property
    def graph_safe(self) -> bool:
        """False when a decode step reads sizes back to the host or branches on per-request state
        (gathered-page attention, the gpt-oss expert loop, cross-attention states), which a CUDA
        graph cannot capture."""
        return not (self.alibi or self.attn_sinks or bool(self.cross_layers))

    def layer_window(self, layer: int) -> int:
        if self.sliding_window <= 0:
            return 0
        if self.layer_types:
            return self.sliding_window if self.layer_types[layer] == "sliding_attention" else 0
        if self.sliding_window_pattern > 0 and (layer + 1) % self.sliding_window_pattern == 0:
            return 0
        return self.sliding_window

    def param_count(self) -> int:
        h, l = self.hidden_size, self.num_layers
        attn = h * (self.q_size + 2 * self.kv_size) + self.q_size * h
        if self.mla is not None:
            m = self.mla
            qd = m.qk_nope_head_dim + m.qk_rope_head_dim
            attn = (h * m.q_lora_rank + m.q_lora_rank * self.num_heads * qd if m.q_lora_rank else h * self.num_heads * qd)
            attn += h * (m.kv_lora_rank + m.qk_rope_head_dim)
            attn += m.kv_lora_rank * self.num_heads * (m.qk_nope_head_dim + m.v_head_dim)
            attn += self.num_heads * m.v_head_dim * h
        total = 0
        for i in range(l):
            if self.layer_is_moe(i):
                mo = self.moe
                ffn = mo.num_experts * 3 * h * mo.expert_ffn + mo.num_shared_experts * 3 * h * (mo.shared_ffn or mo.expert_ffn) + h * mo.num_experts
            else:
                ffn = (3 if self.gated_ffn else 2) * h * self.ffn_size
            total += attn + ffn + 2 * h
        total += self.vocab_size * h * (1 if self.tie_embeddings else 2) + h
        return total

    def validate_tp(self, tp: int) -> None:
        """Same divisibility rules as the reference's TensorParallelTransformer.ValidateConfig
        (src/HartsyInference.LLM/Transformer/TensorParallelTransformer.cs:59-108)."""
        if tp <= 1:
            return
        if self.num_heads % tp or self.ffn_size % tp:
            raise ValueError(f"heads ({self.num_heads}) and ffn ({self.ffn_size}) must divide by tp={tp}")
        if self.num_kv_heads % tp and tp % self.num_kv_heads:
            raise ValueError(f"kv heads ({self.num_kv_heads}) incompatible with tp={tp}")


# ---------------------------------------------------------------------------------------------
PRESETS: dict[str, TransformerConfig] = {
    # Qwen2.5-0.5B: 24 layers, hidden 896, 14 q / 2 kv heads x 64, FFN 4864, tied embeddings
    "qwen2.5-0.5b": TransformerConfig(
        arch="qwen2", vocab_size=151936, hidden_size=896, num_layers=24, num_heads=14, num_kv_heads=2,
        head_dim=64, ffn_size=4864, rms_eps=1e-6, rope_theta=1e6, tie_embeddings=True, qkv_bias=True,
        max_position=32768, bos_token_id=151643, eos_token_ids=(151645, 151643)),
    "llama-3-8b": TransformerConfig(
        arch="llama", vocab_size=128256, hidden_size=4096, num_layers=32, num_heads=32, num_kv_heads=8,
        head_dim=128, ffn_size=14336, rms_eps=1e-5, rope_theta=5e5, max_position=8192,
        bos_token_id=128000, eos_token_ids=(128001, 128009)),
    # Llama-3-70B: 80 layers, hidden 8192, 64 q / 8 kv heads x 128, FFN 28672, vocab 128256
    "llama-3-70b": TransformerConfig(
        arch="llama", vocab_size=128256, hidden_size=8192, num_layers=80, num_heads=64, num_kv_heads=8,
        head_dim=128, ffn_size=28672, rms_eps=1e-5, rope_theta=5e5, max_position=8192,
        bos_token_id=128000, eos_token_ids=(128001, 128009)),
    # DeepSeek-V3: 61 layers (3 dense, FFN 18432), hidden 7168, MLA, 256 routed experts FFN 2048 + 1 shared
    "deepseek-v3": TransformerConfig(
        arch="deepseek3", vocab_size=129280, hidden_size=7168, num_layers=61, num_heads=128, num_kv_heads=128,
        head_dim=192, ffn_size=18432, rms_eps=1e-6, rope_theta=10000.0, rope_style=1, max_position=163840,
        moe=MoeConfig(num_experts=256, top_k=8, expert_ffn=2048, num_shared_experts=1, shared_ffn=2048,
                      scoring="sigmoid", norm_topk_prob=True, routed_scaling_factor=2.5, n_group=8,
                      topk_group=4, use_correction_bias=True, first_dense_layers=3),
        mla=MlaConfig(q_lora_rank=1536, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64,
                      v_head_dim=128),
        bos_token_id=0, eos_token_ids=(1,)),
}


def tiny(base: str = "qwen2.5-0.5b", **over: Any) -> TransformerConfig:
    """A scaled-down config of the same architecture for tests (same code paths, toy sizes)."""
    cfg = PRESETS[base]
    small = dict(vocab_size=512, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=64,
                 ffn_size=512, max_position=2048)
    small.update(over)
    return replace(cfg, **small)


def from_hf_config(d: dict) -> TransformerConfig:
    """Map a Hugging Face ``config.json`` (llama / mistral / qwen2 / qwen3 / gemma 1-3 / granite / olmo2 /
    phi3 / glm / glm4 / starcoder2 / stablelm / cohere / cohere2 / nemotron / gpt_neox / gpt2 / granitemoe / mllama (text) / qwen2_vl - qwen2_5_vl - qwen3_vl (text) / hunyuan_v1_dense / apertus / bloom / gpt_oss / gptj / opt / phi / olmo3 / exaone4 / helium / ernie4_5 / arcee / smollm3 / ministral / seed_oss / minicpm / internlm2 / deepseek_v2-v3 / glm4_moe / dots1 / ernie4_5_moe / hunyuan_v1_moe / cwm / gpt_bigcode / falcon / mixtral /
    olmoe / qwen2_moe / qwen3_moe families) onto :class:`TransformerConfig`."""
    mt = d.get("model_type", "llama")
    if mt == "opt":
        d = {**d, "intermediate_size": d.get("ffn_dim") or 4 * d["hidden_size"], "hidden_act": d.get("activation_function", "relu"),
             "tie_word_embeddings": d.get("tie_word_embeddings", True)}
    if mt == "gptj":
        d = {**d, "hidden_size": d["n_embd"], "num_hidden_layers": d["n_layer"], "num_attention_heads": d["n_head"],
             "max_position_embeddings": d.get("n_positions", 2048), "intermediate_size": d.get("n_inner") or 4 * d["n_embd"],
             "hidden_act": d.get("activation_function", "gelu_new"), "tie_word_embeddings": d.get("tie_word_embeddings", False)}
    if mt == "bloom":
        d = {**d, "num_hidden_layers": d["n_layer"], "num_attention_heads": d["n_head"], "intermediate_size": 4 * d["hidden_size"],
             "max_position_embeddings": d.get("seq_length", 2048), "hidden_act": "gelu_new", "rms_norm_eps": d.get("layer_norm_epsilon", 1e-5),
             "tie_word_embeddings": d.get("tie_word_embeddings", True)}
    if mt in ("gpt2", "gpt_bigcode"):          # GPT-2 names its sizes differently
        d = {**d, "hidden_size": d["n_embd"], "num_hidden_layers": d["n_layer"], "num_attention_heads": d["n_head"],
             "max_position_embeddings": d.get("n_positions", 1024), "intermediate_size": d.get("n_inner") or 4 * d["n_embd"],
             "hidden_act": d.get("activation_function", "gelu_new"), "tie_word_embeddings": d.get("tie_word_embeddings", True)}
    heads = d["num_attention_heads"]
    hidden = d["hidden_size"]
    head_dim = d.get("head_dim") or hidden // heads
    rs = d.get("rope_scaling") or d.get("rope_parameters") or {}
    local_theta = float(d.get("rope_local_base_freq") or 0.0)
    if "full_attention" in rs:            # per-layer-type rotary parameters (Gemma 3)
        local_theta = float((rs.get("sliding_attention") or {}).get("rope_theta", local_theta) or 0.0)
        rs = rs["full_attention"] or {}
    kind = rs.get("rope_type", rs.get("type", "none")) if rs else "none"
    scaling = RopeScaling(kind=kind if kind in ("linear", "llama3", "yarn") else "none",
                          factor=float(rs.get("factor", 1.0)),
                          low_freq_factor=float(rs.get("low_freq_factor", 1.0)),
                          high_freq_factor=float(rs.get("high_freq_factor", 4.0)),
                          original_max_position=int(rs.get("original_max_position_embeddings", 8192)),
                          beta_fast=float(rs.get("beta_fast", 32.0)), beta_slow=float(rs.get("beta_slow", 1.0)),
                          attn_factor=float(rs.get("attn_factor", rs.get("mscale", 1.0)) or 1.0),
                          truncate=bool(rs.get("truncate", True)))
    eos = d.get("eos_token_id", 2)
    eos = tuple(eos) if isinstance(eos, (list, tuple)) else (eos,)
    kw: dict[str, Any] = dict(
        arch=mt, vocab_size=d["vocab_size"], hidden_size=hidden, num_layers=d["num_hidden_layers"],
        num_heads=heads, num_kv_heads=d.get("num_key_value_heads", heads), head_dim=head_dim,
        ffn_size=d.get("intermediate_size") or 4 * hidden,
        rms_eps=float(next((d[k] for k in ("rms_norm_eps", "layer_norm_eps", "norm_epsilon", "norm_eps",
                                           "layer_norm_epsilon") if d.get(k) is not None), 1e-5)),
        rope_theta=float(d.get("rope_theta") or rs.get("rope_theta") or 10000.0), rope_scaling=scaling,
        max_position=d.get("max_position_embeddings", 8192),
        tie_embeddings=bool(d.get("tie_word_embeddings", False)),
        qkv_bias=bool(d.get("attention_bias", mt in ("qwen2", "qwen2_moe"))),
        bos_token_id=d.get("bos_token_id", 1) or 0, eos_token_ids=eos)
    prf = d.get("partial_rotary_factor", rs.get("partial_rotary_factor") if rs else None)
    if prf and float(prf) < 1.0:
        kw["rope_dim"] = int(head_dim * float(prf))
    if mt in ("qwen3", "qwen3_moe", "olmo2", "olmoe"):
        kw["qk_norm"] = True
        kw["qkv_bias"] = bool(d.get("attention_bias", False))
    if mt in ("olmo2", "olmo3", "olmoe"):
        kw["qk_norm_full"] = True
        kw["qk_norm"] = True
    if mt in ("olmo2", "olmo3", "exaone4"):
        kw.update(pre_norm=False, post_norms=True)
    if mt == "hunyuan_v1_dense":
        kw.update(qk_norm=bool(d.get("use_qk_norm", True)), qk_norm_after_rope=True)
        alpha = float(rs.get("alpha") or 0.0)
        if alpha > 0:                             # NTK-alpha: a larger rotary base instead of scaled positions
            kw["rope_theta"] = kw["rope_theta"] * alpha ** (head_dim / (head_dim - 2))
    if mt in ("qwen2_vl", "qwen2_vl_text", "qwen2_5_vl", "qwen2_5_vl_text"):
        kw.update(qkv_bias=True, mrope_section=tuple(int(v) for v in rs.get("mrope_section") or ()))
    if mt in ("qwen3_vl", "qwen3_vl_text"):
        kw.update(qk_norm=True, qkv_bias=bool(d.get("attention_bias", False)),
                  mrope_section=tuple(int(v) for v in rs.get("mrope_section") or (24, 20, 20)),
                  mrope_interleaved=bool(rs.get("mrope_interleaved", True)))
    if mt in ("mllama", "mllama_text_model"):
        kw["cross_layers"] = tuple(int(v) for v in d.get("cross_attention_layers") or ())
    if mt == "apertus":       # non-gated xIELU MLP, per-head q/k norm
        kw.update(gated_ffn=False, qk_norm=True)
    if mt == "exaone4":
        kw["qk_norm"] = True                      # per head, before the rotary embedding
    if mt in ("olmo3", "exaone4", "ministral", "smollm3"):
        kw.update(sliding_window=int(d.get("sliding_window") or 0), layer_types=tuple(d.get("layer_types") or ()))
    if mt == "exaone4" and kw.get("sliding_window"):
        kw["nope_global"] = True                  # hybrid models: full-attention layers carry no rotary embedding
    if mt == "olmo":
        kw.update(norm_type="layernorm", rms_eps=1e-5)        # parameter-free LayerNorm
    if mt in ("helium", "ernie4_5"):
        kw["rope_style"] = 1                      # interleaved rotary pairs
    if mt == "arcee":
        kw.update(gated_ffn=False)                # relu^2 MLP without a gate
    if mt == "smollm3" and d.get("no_rope_layers"):
        kw["rope_layers"] = tuple(int(v) for v in d["no_rope_layers"])       # 1 = rotary, 0 = none
    if mt.startswith("gemma"):
        kw.update(norm_plus_one=True, embed_scale=hidden ** 0.5, activation="gelu_tanh",
                  logit_softcap=float(d.get("final_logit_softcapping") or 0.0),
                  attn_softcap=float(d.get("attn_logit_softcapping") or 0.0),
                  post_norms=mt in ("gemma2", "gemma3", "gemma3_text"),
                  sliding_window=int(d.get("sliding_window") or 0),
                  sliding_window_pattern=int(d.get("sliding_window_pattern") or (2 if mt == "gemma2" else 6)),
                  layer_types=tuple(d.get("layer_types") or ()),
                  rope_local_theta=local_theta if mt in ("gemma3", "gemma3_text") else 0.0,
                  qk_norm=mt in ("gemma3", "gemma3_text"))
        if d.get("query_pre_attn_scalar"):
            kw["attn_scale"] = float(d["query_pre_attn_scalar"]) ** -0.5
    act = {"silu": "silu", "swish": "silu", "gelu_pytorch_tanh": "gelu_tanh", "gelu_new": "gelu_tanh",
           "gelu_fast": "gelu_tanh", "gelu": "gelu", "relu2": "relu2", "relu": "relu", "xielu": "xielu"}.get(
               d.get("hidden_act") or d.get("hidden_activation") or "", None)
    if act is not None and not mt.startswith("gemma"):
        kw["activation"] = act
    if mt in ("glm", "glm4"):
        kw.update(rope_style=1, qkv_bias=bool(d.get("attention_bias", True)), post_norms=mt == "glm4")
    if mt == "starcoder2":
        ub = bool(d.get("use_bias", True))
        kw.update(norm_type="layernorm", norm_bias=True, gated_ffn=False, qkv_bias=ub, o_bias=ub, ffn_bias=ub,
                  sliding_window=int(d.get("sliding_window") or 0))
    if mt == "stablelm":
        kw.update(norm_type="layernorm", norm_bias=True, qkv_bias=bool(d.get("use_qkv_bias", False)),
                  parallel_residual=bool(d.get("use_parallel_residual", False)),
                  shared_parallel_norm=bool(d.get("use_parallel_residual", False)))
    if mt in ("gpt2", "gpt_bigcode"):
        kw.update(norm_type="layernorm", norm_bias=True, gated_ffn=False, qkv_bias=True, o_bias=True, ffn_bias=True,
                  use_rope=False, learned_positions=True,
                  num_kv_heads=1 if (mt == "gpt_bigcode" and d.get("multi_query", True)) else heads)
    if mt == "cohere2":
        kw.update(sliding_window=int(d.get("sliding_window") or 0), layer_types=tuple(d.get("layer_types") or ()),
                  sliding_window_pattern=int(d.get("sliding_window_pattern") or 4), nope_global=True)
    if mt in ("cohere", "cohere2"):
        kw.update(norm_type="layernorm", parallel_residual=True, shared_parallel_norm=True, rope_style=1,
                  logits_scale=float(d.get("logit_scale", 1.0)), tie_embeddings=bool(d.get("tie_word_embeddings", True)))
    if mt == "nemotron":
        kw.update(norm_type="layernorm", norm_bias=True, norm_plus_one=True, gated_ffn=False,
                  qkv_bias=bool(d.get("attention_bias", False)), o_bias=bool(d.get("attention_bias", False)),
                  ffn_bias=bool(d.get("mlp_bias", False)))
    if mt == "opt":
        if not d.get("do_layer_norm_before", True) or d.get("word_embed_proj_dim", hidden) != hidden:
            raise ValueError("OPT variants with post-LayerNorm blocks or projected embeddings (350m) are not mapped")
        b = bool(d.get("enable_bias", True))
        kw.update(norm_type="layernorm", norm_bias=True, gated_ffn=False, qkv_bias=b, o_bias=b, ffn_bias=b, use_rope=False,
                  learned_positions=True, learned_position_offset=2, num_kv_heads=heads)
    if mt == "gptj":          # one LayerNorm, parallel branches, interleaved rotary on the first rotary_dim channels
        kw.update(norm_type="layernorm", norm_bias=True, gated_ffn=False, qkv_bias=False, o_bias=False, ffn_bias=True,
                  parallel_residual=True, shared_parallel_norm=True, lm_head_bias=True, rope_style=1, num_kv_heads=heads,
                  rope_dim=int(d.get("rotary_dim") or 0))
    if mt == "phi":           # Phi-1 / Phi-2: one LayerNorm feeds the parallel attention and MLP branches
        kw.update(norm_type="layernorm", norm_bias=True, gated_ffn=False, qkv_bias=True, o_bias=True, ffn_bias=True,
                  parallel_residual=True, shared_parallel_norm=True, lm_head_bias=True,
                  num_kv_heads=d.get("num_key_value_heads") or heads)
    if mt == "bloom":         # LayerNorm blocks with biases everywhere, ALiBi instead of positions
        kw.update(norm_type="layernorm", norm_bias=True, gated_ffn=False, qkv_bias=True, o_bias=True, ffn_bias=True,
                  num_kv_heads=heads, use_rope=False, alibi=True, embed_norm=True)
    if mt == "falcon":
        # attention and MLP read the same residual stream in parallel (one shared LayerNorm, or ln_attn / ln_mlp in the
        # 40B-class layout); multi-query or grouped keys / values; rotary (or ALiBi) positions; plain GELU MLP
        new = bool(d.get("new_decoder_architecture", False))
        bias = bool(d.get("bias", False))
        kvh = (d.get("num_kv_heads") or heads) if new else (1 if d.get("multi_query", True) else heads)
        parallel = bool(d.get("parallel_attn", True)) or new
        kw.update(norm_type="layernorm", norm_bias=True, gated_ffn=False, qkv_bias=bias, o_bias=bias, ffn_bias=bias, num_kv_heads=kvh,
                  parallel_residual=parallel, shared_parallel_norm=parallel and not (new and (d.get("num_ln_in_parallel_attn") or 2) == 2),
                  activation="gelu", ffn_size=d.get("ffn_hidden_size") or 4 * hidden)
        if d.get("alibi", False):
            kw.update(use_rope=False, alibi=True)
    if mt == "gpt_neox":
        ab = bool(d.get("attention_bias", True))
        kw.update(norm_type="layernorm", norm_bias=True, gated_ffn=False, qkv_bias=ab, o_bias=ab, ffn_bias=True,
                  parallel_residual=bool(d.get("use_parallel_residual", True)), num_kv_heads=heads)
        if d.get("rotary_pct") and float(d["rotary_pct"]) < 1.0 and not kw.get("rope_dim"):
            kw["rope_dim"] = int(head_dim * float(d["rotary_pct"]))
    if mt == "minicpm":
        # muP-style scaling: embeddings * scale_emb, each block's output * scale_depth / sqrt(layers),
        # logits / (hidden / dim_model_base)
        kw.update(embedding_multiplier=float(d.get("scale_emb", 1.0)),
                  residual_multiplier=float(d.get("scale_depth", 1.0)) / (d["num_hidden_layers"] ** 0.5),
                  logits_scale=float(d.get("dim_model_base", hidden)) / hidden)
    if mt in ("granite", "granitemoe", "granitemoeshared"):
        kw.update(residual_multiplier=float(d.get("residual_multiplier", 1.0)),
                  embedding_multiplier=float(d.get("embedding_multiplier", 1.0)),
                  logits_scale=1.0 / float(d.get("logits_scaling", 1.0)),
                  attn_scale=float(d.get("attention_multiplier", 0.0)))
    if mt in ("mistral",) and d.get("sliding_window"):
        kw["sliding_window"] = int(d["sliding_window"])
    if mt in ("deepseek_v3", "deepseek_v2"):
        kw["arch"] = "deepseek3"
        kw["rope_style"] = 1
        kw["mla"] = MlaConfig(q_lora_rank=d.get("q_lora_rank") or 0, kv_lora_rank=d["kv_lora_rank"],
                              qk_nope_head_dim=d["qk_nope_head_dim"], qk_rope_head_dim=d["qk_rope_head_dim"],
                              v_head_dim=d["v_head_dim"])
        kw["head_dim"] = d["qk_nope_head_dim"] + d["qk_rope_head_dim"]
        kw["moe"] = MoeConfig(num_experts=d.get("n_routed_experts", 0), top_k=d.get("num_experts_per_tok", 0),
                              expert_ffn=d.get("moe_intermediate_size", 0),
                              num_shared_experts=d.get("n_shared_experts", 0) or 0,
                              shared_ffn=d.get("moe_intermediate_size", 0),
                              scoring=d.get("scoring_func") or ("sigmoid" if mt == "deepseek_v3" else "softmax"),
                              norm_topk_prob=bool(d.get("norm_topk_prob", False)),
                              routed_scaling_factor=float(d.get("routed_scaling_factor", 1.0)),
                              n_group=d.get("n_group", 1) or 1, topk_group=d.get("topk_group", 1) or 1,
                              use_correction_bias=(d.get("topk_method") or ("noaux_tc" if mt == "deepseek_v3" else "")) == "noaux_tc",
                              first_dense_layers=d.get("first_k_dense_replace", 0))
    if mt in ("glm4_moe", "dots1"):
        # routed experts of the DeepSeek-V3 kind (sigmoid scores, selection bias, grouped top-k, shared experts, leading
        # dense layers) on ordinary grouped-query attention with per-head q / k norms
        kw["qk_norm"] = bool(d.get("use_qk_norm", mt == "dots1"))
        kw["qkv_bias"] = bool(d.get("attention_bias", False))
        kw["moe"] = MoeConfig(num_experts=d.get("n_routed_experts", 0), top_k=d.get("num_experts_per_tok", 0),
                              expert_ffn=d.get("moe_intermediate_size", 0), num_shared_experts=d.get("n_shared_experts", 0) or 0,
                              shared_ffn=d.get("moe_intermediate_size", 0), scoring="sigmoid",
                              norm_topk_prob=bool(d.get("norm_topk_prob", True)),
                              routed_scaling_factor=float(d.get("routed_scaling_factor", 1.0)),
                              n_group=d.get("n_group", 1) or 1, topk_group=d.get("topk_group", 1) or 1, use_correction_bias=True,
                              first_dense_layers=d.get("first_k_dense_replace", 0))
    if mt == "ernie4_5_moe":
        # softmax scores, selection bias, renormalised top-k, shared experts; dense layers before ``moe_layer_start_index``
        kw["rope_style"] = 1
        shared = int(d.get("moe_num_shared_experts", 0) or 0)
        kw["moe"] = MoeConfig(num_experts=d.get("moe_num_experts", 0), top_k=d.get("moe_k", 2), expert_ffn=d.get("moe_intermediate_size", 0),
                              num_shared_experts=shared, shared_ffn=d.get("moe_intermediate_size", 0), scoring="softmax",
                              norm_topk_prob=True, use_correction_bias=True, first_dense_layers=int(d.get("moe_layer_start_index", 0) or 0))
    if mt == "hunyuan_v1_moe":
        topk = d.get("moe_topk", 1)
        shared = d.get("num_shared_expert", 1)
        kw.update(qk_norm=bool(d.get("use_qk_norm", True)), qk_norm_after_rope=True)
        kw["moe"] = MoeConfig(num_experts=d.get("num_experts", 0) if not isinstance(d.get("num_experts"), list) else d["num_experts"][0],
                              top_k=topk[0] if isinstance(topk, list) else topk, expert_ffn=d.get("moe_intermediate_size") or d.get("intermediate_size", 0),
                              num_shared_experts=shared[0] if isinstance(shared, list) else shared, shared_ffn=d.get("intermediate_size", 0),
                              scoring="softmax", norm_topk_prob=True)
    if mt == "gpt_oss":       # sink logits, biased projections, alternating windows, clamped-SwiGLU experts with biases
        ab = bool(d.get("attention_bias", True))
        kw.update(qkv_bias=ab, o_bias=ab, attn_sinks=True, sliding_window=int(d.get("sliding_window") or 0),
                  layer_types=tuple(d.get("layer_types") or ()))
        kw["moe"] = MoeConfig(num_experts=d.get("num_local_experts", 0), top_k=d.get("num_experts_per_tok", 4),
                              expert_ffn=d.get("intermediate_size", 0), norm_topk_prob=True)
    if mt in ("olmoe", "qwen2_moe", "qwen3_moe", "mixtral", "granitemoe", "granitemoeshared"):
        kw["moe"] = MoeConfig(num_experts=d.get("num_experts", d.get("num_local_experts", 0)),
                              top_k=d.get("num_experts_per_tok", 2),
                              expert_ffn=d.get("moe_intermediate_size", d.get("intermediate_size", 0)),
                              num_shared_experts=1 if (d.get("shared_expert_intermediate_size") or d.get("shared_intermediate_size")) else 0,
                              shared_ffn=d.get("shared_expert_intermediate_size") or d.get("shared_intermediate_size") or 0,
                              shared_gate=mt == "qwen2_moe",
                              norm_topk_prob=bool(d.get("norm_topk_prob", mt in ("mixtral", "granitemoe", "granitemoeshared"))))
    return TransformerConfig(**kw)


_GGUF_ARCH_ALIASES = {"qwen2": "qwen2", "qwen3": "qwen3", "llama": "llama", "gemma": "gemma", "gemma2": "gemma2",
                      "gemma3": "gemma3", "phi3": "phi3", "granite": "granite", "deepseek2": "deepseek3",
                      "olmoe": "olmoe", "qwen2moe": "qwen2_moe", "mistral": "mistral", "glm4": "glm4",
                      "stablelm": "stablelm", "olmo2": "olmo2", "internlm2": "internlm2", "minicpm": "minicpm",
                      "qwen3moe": "qwen3_moe", "starcoder2": "starcoder2", "gptneox": "gpt_neox", "nemotron": "nemotron",
                      "bloom": "bloom"}


def from_gguf_metadata(md: dict) -> TransformerConfig:
    """Map GGUF key/value metadata (``general.architecture`` + ``<arch>.*`` keys) onto the config."""
    arch = md.get("general.architecture", "llama")
    g = lambda k, default=None: md.get(f"{arch}.{k}", default)
    heads = int(g("attention.head_count"))
    hidden = int(g("embedding_length"))
    head_dim = int(g("attention.key_length", hidden // heads))
    tokens = md.get("tokenizer.ggml.tokens")
    vocab = int(g("vocab_size", len(tokens) if tokens is not None else 32000))
    kw: dict[str, Any] = dict(
        arch=_GGUF_ARCH_ALIASES.get(arch, arch), vocab_size=vocab, hidden_size=hidden,
        num_layers=int(g("block_count")), num_heads=heads,
        num_kv_heads=int(g("attention.head_count_kv", heads)), head_dim=head_dim,
        ffn_size=int(g("feed_forward_length", 4 * hidden)),
        rms_eps=float(g("attention.layer_norm_rms_epsilon", g("attention.layer_norm_epsilon", 1e-5))),
        rope_theta=float(g("rope.freq_base", 10000.0)), rope_dim=int(g("rope.dimension_count", 0) or 0),
        max_position=int(g("context_length", 8192)),
        # llama-family GGUF files store q/k permuted for interleaved-pair rotation
        rope_style=1 if arch in ("llama", "mistral", "granite", "deepseek2", "minicpm") else 0,
        qkv_bias=bool(md.get("__has_qkv_bias__", arch in ("qwen2", "qwen2moe", "starcoder2", "gptneox"))),
        qk_norm=arch in ("qwen3", "qwen3moe", "olmo2", "olmoe", "gemma3"),
        tie_embeddings=not bool(md.get("__has_output_weight__", False)),
        bos_token_id=int(md.get("tokenizer.ggml.bos_token_id", 1)),
        eos_token_ids=(int(md.get("tokenizer.ggml.eos_token_id", 2)),))
    if kw["rope_dim"] == head_dim:
        kw["rope_dim"] = 0
    if g("rope.scaling.type") == "linear":
        kw["rope_scaling"] = RopeScaling(kind="linear", factor=float(g("rope.scaling.factor", 1.0)))
    if arch.startswith("gemma"):
        kw.update(norm_plus_one=False, embed_scale=hidden ** 0.5, activation="gelu_tanh",
                  logit_softcap=float(g("final_logit_softcapping", 0.0) or 0.0),
                  attn_softcap=float(g("attn_logit_softcapping", 0.0) or 0.0),
                  sliding_window=int(g("attention.sliding_window", 0) or 0), post_norms=arch != "gemma")
    if arch in ("gemma2", "gemma3"):
        kw["sliding_window_pattern"] = 2 if arch == "gemma2" else 6
        if arch == "gemma3":
            kw["rope_local_theta"] = float(g("rope.local_freq_base", 10000.0))
    if g("attention.scale"):
        kw["attn_scale"] = float(g("attention.scale"))
    if arch == "granite":
        kw.update(residual_multiplier=float(g("residual_scale", 1.0)), embedding_multiplier=float(g("embedding_scale", 1.0)),
                  logits_scale=1.0 / float(g("logit_scale", 1.0) or 1.0))
    if arch in ("olmo2", "olmoe"):
        kw["qk_norm_full"] = True
    if arch == "olmo2":
        kw.update(pre_norm=False, post_norms=True)
    if arch == "stablelm":
        par = bool(g("use_parallel_residual", False))
        kw.update(norm_type="layernorm", norm_bias=True, parallel_residual=par, shared_parallel_norm=par)
    if arch == "starcoder2":
        kw.update(norm_type="layernorm", norm_bias=True, gated_ffn=False, activation="gelu_tanh", o_bias=True, ffn_bias=True)
    if arch == "gptneox":
        kw.update(norm_type="layernorm", norm_bias=True, gated_ffn=False, activation="gelu", o_bias=True, ffn_bias=True,
                  parallel_residual=bool(g("use_parallel_residual", True)))
    if arch == "nemotron":
        kw.update(norm_type="layernorm", norm_bias=True, gated_ffn=False, activation="relu2")
    if arch == "bloom":
        kw.update(norm_type="layernorm", norm_bias=True, gated_ffn=False, activation="gelu_tanh", o_bias=True, ffn_bias=True,
                  use_rope=False, alibi=True, embed_norm=True, tie_embeddings=not md.get("__has_output_weight__", False))
    if g("expert_count"):
        kw["moe"] = MoeConfig(num_experts=int(g("expert_count")), top_k=int(g("expert_used_count", 2)),
                              expert_ffn=int(g("expert_feed_forward_length", kw["ffn_size"])),
                              num_shared_experts=int(g("expert_shared_count", 0) or 0),
                              shared_ffn=int(g("expert_shared_feed_forward_length", g("expert_feed_forward_length", 0)) or 0),
                              scoring="sigmoid" if int(g("expert_gating_func", 1) or 1) == 2 else "softmax",
                              norm_topk_prob=bool(g("expert_weights_norm", False)),
                              routed_scaling_factor=float(g("expert_weights_scale", 1.0) or 1.0),
                              n_group=int(g("expert_group_count", 1) or 1),
                              topk_group=int(g("expert_group_used_count", 1) or 1),
                              use_correction_bias=bool(md.get("__has_expert_bias__", False)),
                              shared_gate=arch == "qwen2moe",
                              first_dense_layers=int(g("leading_dense_block_count", 0) or 0))
    if g("attention.kv_lora_rank"):
        kw["head_dim"] = int(g("attention.key_length", 192))
        kw["mla"] = MlaConfig(q_lora_rank=int(g("attention.q_lora_rank", 0) or 0),
                              kv_lora_rank=int(g("attention.kv_lora_rank")),
                              qk_rope_head_dim=int(g("rope.dimension_count", 64)),
                              qk_nope_head_dim=int(g("attention.key_length", 192)) - int(g("rope.dimension_count", 64)),
                              v_head_dim=int(g("attention.value_length", 128)))
    return TransformerConfig(**kw)
