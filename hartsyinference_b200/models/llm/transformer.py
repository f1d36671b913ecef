"""Config-driven decoder transformer over the fused ops.

One class runs every dense decoder architecture of :mod:`.config` (llama, mistral, qwen2/3, gemma
1-3, granite, glm4, olmo2, ...), single-GPU or tensor-parallel. Activations are bf16, weights bf16
or 128x128 block-scaled e4m3; the KV cache is a page pool written by the RoPE kernel and read in
place by the attention kernels.

Role in the reference: ``GenericTransformer`` (config-driven decoder, fp32 activations;
src/HartsyInference.LLM/Transformer/GenericTransformer.cs: LoadWeights:171, ForwardEmbeds:409-535,
Layer.Forward:1575-1751, ForwardBatchDecode:856-902, ProjectLogits:931-978) and
``TensorParallelTransformer`` (Megatron split with two all-reduces per layer, ranks executed one
after another by one thread; TensorParallelTransformer.cs:251-341, slicing :529/:552). Here every
rank is its own process and the all-reduce is either NCCL or the fused GEMM+all-reduce kernel.

Layer dataflow (one launch per arrow, residual adds folded into the norm kernel):

    norm(+res) -> qkv GEMM -> [qk-norm] rope + KV page write -> attention -> o GEMM (-> all-reduce)
    norm(+res) -> gate|up GEMM -> GLU (emits fp8 for the next GEMM) -> down GEMM (-> all-reduce)
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Optional

import torch

from ... import config, ops
from ...ops import LinearWeight
from ...parallel.comm import Comm, SingleComm
from .config import RopeScaling, TransformerConfig


@dataclass
class ForwardBatch:
    """Device-side description of one forward pass (a prefill chunk batch or a decode batch)."""
    tokens: torch.Tensor                 # [T] int32
    positions: torch.Tensor              # [T] int32
    slot_mapping: torch.Tensor           # [T] int64, page_index * page + offset, -1 = do not store
    block_table: torch.Tensor            # [S, max_pages] int32
    kv_lens: torch.Tensor                # [S] int32, keys visible to the last query of each sequence
    is_decode: bool
    cu_q: Optional[torch.Tensor] = None  # prefill: [S + 1] int32
    max_q_len: int = 1
    max_kv_len: int = 0
    logit_rows: Optional[torch.Tensor] = None   # prefill: rows (into T) whose logits are needed
    embeds: Optional[torch.Tensor] = None       # optional precomputed input embeddings [T, H]
    positions3: Optional[torch.Tensor] = None       # Qwen-VL: [3, T] int32 time / row / column positions (None: all = positions)
    deepstack: Optional[torch.Tensor] = None        # Qwen3-VL: [taps, T, H] added to the hidden states after the first layers
    cross_states: Optional[object] = None           # Mllama: projected vision states [Tv, H] for every row, or a list
                                                    # with one entry (tensor or None) per sequence
    cross_row_mask: Optional[torch.Tensor] = None   # Mllama: [T], 0 for text rows that precede every image


def build_inv_freq(rot: int, theta: float, scaling: RopeScaling, device) -> tuple[torch.Tensor, float]:
    """Inverse rotary frequencies with linear / llama3 / YaRN scaling, and the attention factor.
    (Reference: src/HartsyInference.Core/Rope/RopeFrequencyBuilder.cs, RopeScaling.cs.)"""
    inv = theta ** (-torch.arange(0, rot, 2, dtype=torch.float64) / rot)
    attn_factor = 1.0
    if scaling.kind == "linear":
        inv = inv / scaling.factor
    elif scaling.kind == "llama3":
        low = scaling.original_max_position / scaling.low_freq_factor
        high = scaling.original_max_position / scaling.high_freq_factor
        wavelen = 2 * math.pi / inv
        smooth = ((scaling.original_max_position / wavelen) - scaling.low_freq_factor) / (
            scaling.high_freq_factor - scaling.low_freq_factor)
        scaled = torch.where(wavelen > low, inv / scaling.factor, inv)
        mid = (wavelen <= low) & (wavelen >= high)
        scaled = torch.where(mid, (1 - smooth) * inv / scaling.factor + smooth * inv, scaled)
        inv = scaled
    elif scaling.kind == "yarn":
        def corr_dim(n_rot):
            return (rot * math.log(scaling.original_max_position / (n_rot * 2 * math.pi))) / (2 * math.log(theta))
        lo, hi = corr_dim(scaling.beta_fast), corr_dim(scaling.beta_slow)
        if scaling.truncate:
            lo, hi = math.floor(lo), math.ceil(hi)
        lo, hi = max(lo, 0), min(hi, rot // 2 - 1)
        ramp = ((torch.arange(rot // 2, dtype=torch.float64) - lo) / max(hi - lo, 1e-3)).clamp(0, 1)
        mask = 1 - ramp
        inv = inv / scaling.factor * (1 - mask) + inv * mask
        attn_factor = scaling.attn_factor * (0.1 * math.log(scaling.factor) + 1.0) if scaling.factor > 1 else 1.0
    return inv.to(torch.float32).to(device), attn_factor


def alibi_slopes(heads: int) -> torch.Tensor:
    """ALiBi head slopes: a geometric sequence for the largest power of two <= heads, then every
    other term of the sequence for twice that count to fill the remainder."""
    n = 1 << (heads.bit_length() - 1)
    base = 2.0 ** (-(2.0 ** -(math.log2(n) - 3)))
    out = [base ** (i + 1) for i in range(n)]
    if n < heads:
        extra = 2.0 ** (-(2.0 ** -(math.log2(2 * n) - 3)))
        out += [extra ** (2 * i + 1) for i in range(heads - n)]
    return torch.tensor(out, dtype=torch.float32)


@dataclass
class LayerWeights:
    in_norm: torch.Tensor
    qkv: LinearWeight
    o: LinearWeight
    post_norm: torch.Tensor
    gate_up: Optional[LinearWeight] = None
    down: Optional[LinearWeight] = None
    q_norm: Optional[torch.Tensor] = None
    k_norm: Optional[torch.Tensor] = None
    post_attn_norm: Optional[torch.Tensor] = None     # sandwich norms (Gemma 2/3)
    post_ffn_norm: Optional[torch.Tensor] = None
    ffn_module: Optional[object] = None               # MoE feed-forward (callable) instead of gate_up/down
    attn_module: Optional[object] = None              # MLA attention (callable) instead of qkv/o
    attn_dp: Optional[object] = None                  # the same attention over ALL heads with replicated weights
                                                      # (data-parallel attention at decode, parallel/dp_attention.py)
    in_norm_b: Optional[torch.Tensor] = None          # LayerNorm biases (StableLM, StarCoder 2, GPT-NeoX, Nemotron)
    post_norm_b: Optional[torch.Tensor] = None
    cross: Optional[object] = None                    # cross-attention layer over vision states (Mllama) instead of a block
    act_params: Optional[tuple] = None                # xIELU: (alpha_p, alpha_n, beta, eps) as floats (Apertus)
    sinks: Optional[torch.Tensor] = None              # per-head sink logit in the attention softmax (gpt-oss)


def x_is_cuda(x) -> bool:
    return (x.data if isinstance(x, ops.Fp8Act) else x).is_cuda


class DecoderModel:
    def __init__(self, cfg: TransformerConfig, device: torch.device | str = "cpu", comm: Optional[Comm] = None,
                 fp8: bool = False, layer_range: Optional[tuple[int, int]] = None, dp_attention: bool = False):
        self.cfg = cfg
        # pipeline stage: this instance holds layers [layer0, layer1) only (all of them by default)
        self.layer0, self.layer1 = layer_range if layer_range is not None else (0, cfg.num_layers)
        self.first_stage, self.last_stage = self.layer0 == 0, self.layer1 == cfg.num_layers
        self.device = torch.device(device)
        self.comm = comm or SingleComm()
        self.tp = self.comm.world
        self.tp_rank = self.comm.rank
        cfg.validate_tp(self.tp)
        self.fp8 = fp8
        self.hq = cfg.num_heads // self.tp
        self.hkv = max(1, cfg.num_kv_heads // self.tp)
        self.ffn = cfg.ffn_size // self.tp
        self.vocab_local = (cfg.vocab_size + self.tp - 1) // self.tp
        self.embed: Optional[torch.Tensor] = None
        self.lm_head: Optional[LinearWeight] = None
        self.final_norm: Optional[torch.Tensor] = None
        self.layers: list[LayerWeights] = []
        rot = cfg.mla.qk_rope_head_dim if cfg.mla is not None else cfg.rotary_dim
        self.inv_freq, self.rope_attn_factor = build_inv_freq(rot, cfg.rope_theta, cfg.rope_scaling, self.device)
        # sliding-window layers of Gemma 3 rotate with their own base and no long-context scaling
        self.inv_freq_local = (build_inv_freq(rot, cfg.rope_local_theta, RopeScaling(), self.device)[0]
                               if cfg.rope_local_theta > 0 else None)
        self.final_norm_b: Optional[torch.Tensor] = None
        self.pos_embed: Optional[torch.Tensor] = None      # learned absolute positions (GPT-2)
        self.embed_norm_w: Optional[torch.Tensor] = None   # LayerNorm on the embedding output (BLOOM)
        self.embed_norm_b: Optional[torch.Tensor] = None
        self.alibi_slopes: Optional[torch.Tensor] = None   # [local heads]
        self.kv_cache: Optional[torch.Tensor] = None
        self.all_reduce: Callable[[torch.Tensor], torch.Tensor] = self.comm.all_reduce
        # hook for the fused GEMM + all-reduce path: (x, weight, residual) -> reduced output
        self.row_parallel_linear: Optional[Callable] = None
        # latency-oriented all-reduce over the symmetric heap (parallel/custom_ar.py): the row-parallel
        # GEMM writes into its input buffer, tensors that do not fit go through ``all_reduce``
        self.custom_ar = None
        # fused row-parallel linear + all-reduce + residual + RMSNorm (+ fp8 emit) kernel
        # (parallel/fused.py::FusedRowParallel); drives the whole layer loop of small batches
        self.fused_rp = None
        # data-parallel attention at decode (latent-attention MoE models, tp > 1): every layer also holds
        # the attention weights of all heads; ``dp_exchange`` (parallel/dp_attention.py) moves the tokens
        self.dp_attention = bool(dp_attention) and cfg.mla is not None and self.tp > 1 and layer_range is None
        self.dp_exchange = None

    # ------------------------------------------------------------------------------ weights
    def _lw(self, w: torch.Tensor, bias: Optional[torch.Tensor] = None, allow_fp8: bool = True) -> LinearWeight:
        w = w.to(self.device)
        b = None if bias is None else bias.to(self.device)
        return LinearWeight.from_dense(w, b, fp8=self.fp8 and allow_fp8)

    def kv_head_slice(self) -> slice:
        """KV heads owned by this rank (replicated across ranks when tp > num_kv_heads)."""
        hkv_total = self.cfg.num_kv_heads
        if self.tp <= hkv_total:
            return slice(self.tp_rank * self.hkv, (self.tp_rank + 1) * self.hkv)
        rep = self.tp // hkv_total
        idx = self.tp_rank // rep
        return slice(idx, idx + 1)

    def load_state_dict(self, get: Callable[[str], Optional[torch.Tensor]]) -> None:
        """Load Hugging Face-named tensors (``model.layers.N.self_attn.q_proj.weight`` ...), slicing
        each tensor to this rank's shard. ``get(name)`` returns a CPU tensor or None."""
        cfg, d = self.cfg, self.cfg.head_dim
        r, tp = self.tp_rank, self.tp
        dt = torch.bfloat16

        def need(name):
            t = get(name)
            if t is None:
                raise KeyError(f"missing tensor {name}")
            return t

        emb = need("model.embed_tokens.weight")
        self.embed = emb.to(dt).to(self.device)
        head = get("lm_head.weight")
        if head is None or cfg.tie_embeddings:
            head = emb
        v0, v1 = r * self.vocab_local, min(cfg.vocab_size, (r + 1) * self.vocab_local)
        hw = head[v0:v1]
        if hw.shape[0] < self.vocab_local:   # pad the last shard so every rank has the same shape
            hw = torch.cat([hw, torch.zeros(self.vocab_local - hw.shape[0], hw.shape[1], dtype=hw.dtype)])
        hb = None
        if cfg.lm_head_bias and get("lm_head.bias") is not None:
            hb = get("lm_head.bias")[v0:v1]
            if hb.shape[0] < self.vocab_local:
                hb = torch.cat([hb, torch.zeros(self.vocab_local - hb.shape[0], dtype=hb.dtype)])
            hb = hb.to(dt)
        self.lm_head = self._lw(hw.to(dt), hb, allow_fp8=False)
        self.final_norm = need("model.norm.weight").to(dt).to(self.device)
        dev = lambda t_: None if t_ is None else t_.to(dt).to(self.device)
        self.final_norm_b = dev(get("model.norm.bias")) if cfg.norm_bias else None
        if cfg.embed_norm:
            self.embed_norm_w, self.embed_norm_b = dev(need("model.embed_norm.weight")), dev(get("model.embed_norm.bias"))
        if cfg.alibi:
            self.alibi_slopes = alibi_slopes(cfg.num_heads)[self.tp_rank * self.hq:(self.tp_rank + 1) * self.hq].to(self.device)
        if cfg.learned_positions:
            self.pos_embed = dev(need("model.embed_positions.weight"))
        if cfg.qk_norm_full and tp > 1:
            raise ValueError("q/k normalisation over the whole projection is not sharded; load this model with tp=1")
        kvs = self.kv_head_slice()
        self.layers = []

        def row_bias(name):            # the bias of a row-parallel linear is added once, by rank 0
            b = get(name)
            if b is None:
                return None
            return (b if r == 0 else torch.zeros_like(b)).to(dt)

        for i in range(self.layer0, self.layer1):
            p = f"model.layers.{i}."
            if i in cfg.cross_layers:
                from .mllama import CrossLayer
                full = lambda n: self._lw(need(p + n).contiguous().to(dt), None)      # replicated on every rank
                gu = torch.cat([need(p + "mlp.gate_proj.weight"), need(p + "mlp.up_proj.weight")]).to(dt)
                lw = LayerWeights(in_norm=None, qkv=None, o=None, post_norm=None)
                lw.cross = CrossLayer(dev(need(p + "input_layernorm.weight")), dev(need(p + "post_attention_layernorm.weight")),
                                      full("cross_attn.q_proj.weight"), full("cross_attn.k_proj.weight"),
                                      full("cross_attn.v_proj.weight"), full("cross_attn.o_proj.weight"),
                                      dev(need(p + "cross_attn.q_norm.weight")), dev(need(p + "cross_attn.k_norm.weight")),
                                      self._lw(gu, None), full("mlp.down_proj.weight"),
                                      float(torch.tanh(need(p + "cross_attn_attn_gate").float()).reshape(-1)[0]),
                                      float(torch.tanh(need(p + "cross_attn_mlp_gate").float()).reshape(-1)[0]),
                                      cfg.num_heads, cfg.num_kv_heads, d, cfg.rms_eps)
                self.layers.append(lw)
                continue
            is_moe = cfg.moe is not None and cfg.moe.num_experts > 0 and i >= cfg.moe.first_dense_layers
            post_name = "post_attention_layernorm"
            if cfg.shared_parallel_norm:
                post_name = "input_layernorm"
            lw = LayerWeights(
                in_norm=dev(need(p + "input_layernorm.weight")) if cfg.pre_norm else None,
                qkv=None, o=None,
                post_norm=dev(need(p + post_name + ".weight")))
            if cfg.norm_bias:
                lw.in_norm_b = dev(get(p + "input_layernorm.bias"))
                lw.post_norm_b = dev(get(p + post_name + ".bias"))
            if cfg.mla is not None:
                lw.attn_module = self._load_mla(need, get, p + "self_attn.")
                lw.attn_dp, self._attn_dp_pending = getattr(self, "_attn_dp_pending", None), None
            else:
                q = need(p + "self_attn.q_proj.weight")[r * self.hq * d:(r + 1) * self.hq * d]
                k = need(p + "self_attn.k_proj.weight")[kvs.start * d:kvs.stop * d]
                v = need(p + "self_attn.v_proj.weight")[kvs.start * d:kvs.stop * d]
                qkv_b = None
                if cfg.qkv_bias and get(p + "self_attn.q_proj.bias") is not None:
                    qkv_b = torch.cat([need(p + "self_attn.q_proj.bias")[r * self.hq * d:(r + 1) * self.hq * d],
                                       need(p + "self_attn.k_proj.bias")[kvs.start * d:kvs.stop * d],
                                       need(p + "self_attn.v_proj.bias")[kvs.start * d:kvs.stop * d]])
                o = need(p + "self_attn.o_proj.weight")[:, r * self.hq * d:(r + 1) * self.hq * d]
                lw.qkv = self._lw(torch.cat([q, k, v]).to(dt), None if qkv_b is None else qkv_b.to(dt))
                lw.o = self._lw(o.contiguous().to(dt), row_bias(p + "self_attn.o_proj.bias") if cfg.o_bias else None)
            if cfg.attn_sinks:
                lw.sinks = dev(need(p + "self_attn.sinks"))[r * self.hq:(r + 1) * self.hq].float()
            if is_moe and cfg.arch == "gpt_oss":
                from .gpt_oss import GptOssMoe, expert_tensor
                lw.ffn_module = GptOssMoe(dev(need(p + "mlp.router.weight").to(dt)), dev(need(p + "mlp.router.bias").to(dt)),
                                          dev(expert_tensor(get, p + "mlp.experts.gate_up_proj").to(dt)), dev(need(p + "mlp.experts.gate_up_proj_bias").to(dt)),
                                          dev(expert_tensor(get, p + "mlp.experts.down_proj").to(dt)), dev(need(p + "mlp.experts.down_proj_bias").to(dt)),
                                          cfg.moe.top_k)
            elif is_moe:
                lw.ffn_module = self._load_moe(need, get, p)
            else:
                fs = slice(r * self.ffn, (r + 1) * self.ffn)
                up = need(p + "mlp.up_proj.weight")[fs]
                down = need(p + "mlp.down_proj.weight")[:, fs]
                ub = get(p + "mlp.up_proj.bias") if cfg.ffn_bias else None
                if cfg.gated_ffn:
                    gate = need(p + "mlp.gate_proj.weight")[fs]
                    gb = get(p + "mlp.gate_proj.bias") if cfg.ffn_bias else None
                    gub = torch.cat([gb[fs], ub[fs]]).to(dt) if gb is not None and ub is not None else None
                    lw.gate_up = self._lw(torch.cat([gate, up]).to(dt), gub)
                else:
                    lw.gate_up = self._lw(up.contiguous().to(dt), None if ub is None else ub[fs].to(dt))
                lw.down = self._lw(down.contiguous().to(dt), row_bias(p + "mlp.down_proj.bias") if cfg.ffn_bias else None)
            if cfg.activation == "xielu":
                sp = torch.nn.functional.softplus
                beta = float(need(p + "mlp.act_fn.beta").float().reshape(-1)[0])
                lw.act_params = (float(sp(need(p + "mlp.act_fn.alpha_p").float()).reshape(-1)[0]),
                                 beta + float(sp(need(p + "mlp.act_fn.alpha_n").float()).reshape(-1)[0]),
                                 beta, float(need(p + "mlp.act_fn.eps").float().reshape(-1)[0]))
            if cfg.qk_norm:
                qn, kn = need(p + "self_attn.q_norm.weight"), need(p + "self_attn.k_norm.weight")
                if cfg.norm_plus_one:      # Gemma 3 stores w - 1 for these too; the rotary kernel multiplies by w
                    qn, kn = qn.float() + 1.0, kn.float() + 1.0
                lw.q_norm, lw.k_norm = qn.to(dt).to(self.device), kn.to(dt).to(self.device)
            if cfg.post_norms:
                lw.post_attn_norm = lw.post_norm
                lw.post_norm = dev(need(p + "pre_feedforward_layernorm.weight")) if cfg.pre_norm else None
                lw.post_ffn_norm = dev(need(p + "post_feedforward_layernorm.weight"))
            self.layers.append(lw)

    def _load_mla(self, need, get, p: str):
        """Hugging Face DeepSeek attention tensors -> absorbed, head-sharded MLA weights."""
        from .mla import MlaAttention, MlaWeights, fold_q, split_kv_b
        cfg, m, dt = self.cfg, self.cfg.mla, torch.bfloat16
        r, hl = self.tp_rank, self.hq
        dq = m.qk_nope_head_dim + m.qk_rope_head_dim
        dev = lambda t_: t_.to(dt).to(self.device)
        fold = self.device.type == "cuda" and bool(config.get("mla_fold_q"))
        q_name = p + ("q_b_proj.weight" if m.q_lora_rank else "q_proj.weight")
        if m.q_lora_rank:
            q_a = self._lw(need(p + "q_a_proj.weight").to(dt))
            q_a_norm = dev(need(p + "q_a_layernorm.weight"))
        else:
            q_a, q_a_norm = None, None
        q_b_dense = need(q_name)[r * hl * dq:(r + 1) * hl * dq].to(dt)
        q_b = self._lw(q_b_dense)
        per = m.qk_nope_head_dim + m.v_head_dim
        kv_b = need(p + "kv_b_proj.weight")[r * hl * per:(r + 1) * hl * per].to(dt)
        w_uk, w_uv = split_kv_b(kv_b, hl, m.qk_nope_head_dim, m.v_head_dim)

        def folded(qb, uk, heads):
            return self._lw(fold_q(qb.to(self.device), uk.to(self.device), heads, m.qk_nope_head_dim, m.qk_rope_head_dim)) if fold else None

        w = MlaWeights(
            q_a=q_a, q_a_norm=q_a_norm, q_b=q_b,
            kv_a=self._lw(need(p + "kv_a_proj_with_mqa.weight").to(dt), allow_fp8=False),
            kv_a_norm=dev(need(p + "kv_a_layernorm.weight")),
            w_uk=self._lw(w_uk, allow_fp8=False), w_uv=self._lw(w_uv, allow_fp8=False),
            o=self._lw(need(p + "o_proj.weight")[:, r * hl * m.v_head_dim:(r + 1) * hl * m.v_head_dim]
                       .contiguous().to(dt)),
            q_fold=folded(q_b_dense, w_uk, hl))
        if self.dp_attention:
            heads = cfg.num_heads
            uk, uv = split_kv_b(need(p + "kv_b_proj.weight").to(dt), heads, m.qk_nope_head_dim, m.v_head_dim)
            full = MlaWeights(q_a=w.q_a, q_a_norm=w.q_a_norm, q_b=self._lw(need(q_name).to(dt)),
                              kv_a=w.kv_a, kv_a_norm=w.kv_a_norm, w_uk=self._lw(uk, allow_fp8=False),
                              w_uv=self._lw(uv, allow_fp8=False), o=self._lw(need(p + "o_proj.weight").to(dt)),
                              q_fold=folded(need(q_name).to(dt), uk, heads))
            self._attn_dp_pending = MlaAttention(cfg, full, heads)
            self._attn_dp_pending.reduce_output = False
        return MlaAttention(cfg, w, hl)

    def _load_moe(self, need, get, p: str):
        """Expert tensors of one layer (DeepSeek / Qwen-MoE / OLMoE ``mlp.*`` names or Mixtral
        ``block_sparse_moe.*`` names) -> this rank's stacked expert weights."""
        from .moe import MoeFeedForward, MoeWeights
        cfg, moe, dt = self.cfg, self.cfg.moe, torch.bfloat16
        r, tp = self.tp_rank, self.tp
        e_local = moe.num_experts // tp
        mixtral = get(p + "block_sparse_moe.gate.weight") is not None
        base = p + ("block_sparse_moe." if mixtral else "mlp.")
        names = ("w1", "w3", "w2") if mixtral else ("gate_proj", "up_proj", "down_proj")
        router_w = next((t for t in (get(base + n) for n in ("gate.weight", "gate.wg.weight", "router.weight")) if t is not None), None)
        router = LinearWeight((router_w if router_w is not None else need(base + "gate.weight")).to(dt).to(self.device))
        bias = get(base + "gate.e_score_correction_bias")
        if bias is None:
            bias = get(base + "gate.moe_statics.e_score_correction_bias")
            bias = None if bias is None else bias.reshape(-1)
        gus, dns = [], []
        stacked_gu, stacked_dn = get(base + "experts.gate_up_proj"), get(base + "experts.down_proj")
        for e in range(r * e_local, (r + 1) * e_local):
            if stacked_gu is not None:        # one [E, 2F, H] / [E, H, F] tensor per layer
                gus.append(stacked_gu[e].to(dt))
                dns.append(stacked_dn[e].to(dt))
                continue
            ep = f"{base}experts.{e}."
            gus.append(torch.cat([need(ep + names[0] + ".weight"), need(ep + names[1] + ".weight")]).to(dt))
            dns.append(need(ep + names[2] + ".weight").to(dt))
        w = MoeWeights(router=router,
                       router_bias=None if bias is None else bias.float().contiguous().to(self.device),
                       gate_up=self._lw(torch.cat(gus)), down=self._lw(torch.cat(dns)))
        for sp in ("shared_experts.", "shared_expert.", "shared_mlp."):
            sg = get(base + sp + "gate_proj.weight")
            if sg is None:
                continue
            fs = sg.shape[0] // tp
            su = need(base + sp + "up_proj.weight")
            sd = need(base + sp + "down_proj.weight")
            w.shared_gate_up = self._lw(torch.cat([sg[r * fs:(r + 1) * fs], su[r * fs:(r + 1) * fs]]).to(dt))
            w.shared_down = self._lw(sd[:, r * fs:(r + 1) * fs].contiguous().to(dt))
            gate = get(base + "shared_expert_gate.weight")
            if gate is not None:
                w.shared_gate = LinearWeight(gate.to(dt).to(self.device))
        return MoeFeedForward(cfg, w, r, tp, all_reduce=lambda y: self.all_reduce(y))

    def random_init(self, seed: int = 0, std: float = 0.02) -> None:
        """Synthetic weights generated on the device (no host copy): bf16 N(0, std), or e4m3 bytes
        with constant block scales that reproduce the same distribution."""
        cfg, d, dev = self.cfg, self.cfg.head_dim, self.device
        counter = [seed * 1000003 + self.tp_rank * 7919]

        def dense(n, k, s=std):
            counter[0] += 1
            t = torch.empty(n, k, dtype=torch.bfloat16, device=dev)
            ops.fill_random_(t, counter[0], s)
            return t

        def lin(n, k, bias=False, allow_fp8=True, seed=None):
            counter[0] += 1
            if seed is not None:          # a tensor that is the same on every rank
                keep, counter[0] = counter[0], seed
                try:
                    return lin(n, k, bias, allow_fp8)
                finally:
                    counter[0] = keep
            if self.fp8 and allow_fp8 and k % 128 == 0:
                w = torch.empty(n, k, dtype=torch.uint8, device=dev)
                ops.fill_random_(w, counter[0])
                sc = torch.full(((n + 127) // 128, k // 128), std / 112.0, dtype=torch.float32, device=dev)
                b = dense(1, n).reshape(n) if bias else None
                return LinearWeight.from_quantized(w, sc, b)
            b = dense(1, n).reshape(n) if bias else None
            return LinearWeight(dense(n, k), None, b)

        ones = lambda n: torch.ones(n, dtype=torch.bfloat16, device=dev)
        # the embedding table is shared by all ranks: seed it independently of the rank
        emb_seed = seed * 1000003 + 17
        self.embed = torch.empty(cfg.vocab_size, cfg.hidden_size, dtype=torch.bfloat16, device=dev)
        ops.fill_random_(self.embed, emb_seed, std)
        if cfg.tie_embeddings:
            v0 = self.tp_rank * self.vocab_local
            hw = self.embed[v0:v0 + self.vocab_local]
            if hw.shape[0] < self.vocab_local:
                hw = torch.cat([hw, torch.zeros(self.vocab_local - hw.shape[0], cfg.hidden_size, dtype=hw.dtype, device=dev)])
            self.lm_head = LinearWeight(hw.contiguous() if self.tp > 1 else hw)
        else:
            self.lm_head = lin(self.vocab_local, cfg.hidden_size, allow_fp8=False)
        self.final_norm = ones(cfg.hidden_size)
        self.layers = []
        for li in range(cfg.num_layers):
            if not (self.layer0 <= li < self.layer1):
                counter[0] += 64          # keep the remaining layers' seeds independent of the stage split
                continue
            counter[0] = (seed * 1000003 + self.tp_rank * 7919) + 1000 + li * 64
            is_moe = cfg.moe is not None and cfg.moe.num_experts > 0 and li >= cfg.moe.first_dense_layers
            lw = LayerWeights(
                in_norm=ones(cfg.hidden_size),
                qkv=None if cfg.mla is not None else lin((self.hq + 2 * self.hkv) * d, cfg.hidden_size, bias=cfg.qkv_bias),
                o=None if cfg.mla is not None else lin(cfg.hidden_size, self.hq * d),
                post_norm=ones(cfg.hidden_size),
                gate_up=None if is_moe else lin(2 * self.ffn, cfg.hidden_size),
                down=None if is_moe else lin(cfg.hidden_size, self.ffn))
            if is_moe:
                lw.ffn_module = self._random_moe(lin, dense)
            if cfg.mla is not None:
                lw.attn_module = self._random_mla(lin, ones)
                lw.attn_dp, self._attn_dp_pending = getattr(self, "_attn_dp_pending", None), None
            if cfg.qk_norm:
                lw.q_norm, lw.k_norm = ones(d), ones(d)
            if cfg.post_norms:
                lw.post_attn_norm, lw.post_ffn_norm = ones(cfg.hidden_size), ones(cfg.hidden_size)
            self.layers.append(lw)

    def _random_moe(self, lin, dense):
        from .moe import MoeFeedForward, MoeWeights
        cfg, moe, dev = self.cfg, self.cfg.moe, self.device
        e_local = moe.num_experts // self.tp
        router = LinearWeight(torch.empty(moe.num_experts, cfg.hidden_size, dtype=torch.bfloat16, device=dev))
        # the router is replicated: seed it independently of the rank
        self._shared_seed = getattr(self, "_shared_seed", 7_000_003) + 1
        ops.fill_random_(router.weight, self._shared_seed, 0.05)
        bias = None
        if moe.use_correction_bias:
            b = torch.empty(1, moe.num_experts, dtype=torch.bfloat16, device=dev)
            ops.fill_random_(b, self._shared_seed + 500_000, 0.01)
            bias = b.float().reshape(-1).contiguous()
        w = MoeWeights(router=router, router_bias=bias,
                       gate_up=lin(e_local * 2 * moe.expert_ffn, cfg.hidden_size),
                       down=lin(e_local * cfg.hidden_size, moe.expert_ffn))
        if moe.num_shared_experts > 0:
            fs = moe.shared_ffn * moe.num_shared_experts // self.tp
            w.shared_gate_up = lin(2 * fs, cfg.hidden_size)
            w.shared_down = lin(cfg.hidden_size, fs)
        return MoeFeedForward(cfg, w, self.tp_rank, self.tp, all_reduce=lambda y: self.all_reduce(y))

    def _random_mla(self, lin, ones):
        from .mla import MlaAttention, MlaWeights
        cfg, m = self.cfg, self.cfg.mla
        hl = self.hq
        dq = m.qk_nope_head_dim + m.qk_rope_head_dim
        if self.dp_attention:
            return self._random_mla_dp(lin, ones)
        w = MlaWeights(
            q_a=lin(m.q_lora_rank, cfg.hidden_size) if m.q_lora_rank else None,
            q_a_norm=ones(m.q_lora_rank) if m.q_lora_rank else None,
            q_b=lin(hl * dq, m.q_lora_rank if m.q_lora_rank else cfg.hidden_size),
            kv_a=lin(m.kv_lora_rank + m.qk_rope_head_dim, cfg.hidden_size, allow_fp8=False),
            kv_a_norm=ones(m.kv_lora_rank),
            w_uk=lin(hl * m.kv_lora_rank, m.qk_nope_head_dim, allow_fp8=False),
            w_uv=lin(hl * m.v_head_dim, m.kv_lora_rank, allow_fp8=False),
            o=lin(cfg.hidden_size, hl * m.v_head_dim))
        if self.device.type == "cuda" and config.get("mla_fold_q"):
            # synthetic weights: the folded projection is drawn by itself (prefill chunks above 256 rows use
            # q_b + W_uk, a different random function of the input; timing is what such a model is for)
            w.q_fold = lin(hl * (m.kv_lora_rank + m.qk_rope_head_dim), m.q_lora_rank if m.q_lora_rank else cfg.hidden_size)
        return MlaAttention(cfg, w, hl)

    def _random_mla_dp(self, lin, ones):
        """Attention weights of all heads, the same on every rank (seeded independently of the rank), and
        this rank's head shard for the tensor-parallel prefill path as slices of them, so that prefill
        and decode are the same model."""
        from .mla import MlaAttention, MlaWeights
        cfg, m, r = self.cfg, self.cfg.mla, self.tp_rank
        heads, hl = cfg.num_heads, self.hq
        dq = m.qk_nope_head_dim + m.qk_rope_head_dim

        def shared(n, k, allow_fp8=True):      # the factory's own counter depends on the rank
            self._replicated_seed = getattr(self, "_replicated_seed", 9_000_001) + 2
            return lin(n, k, allow_fp8=allow_fp8, seed=self._replicated_seed)

        q_in = m.q_lora_rank if m.q_lora_rank else cfg.hidden_size
        full = MlaWeights(
            q_a=shared(m.q_lora_rank, cfg.hidden_size) if m.q_lora_rank else None,
            q_a_norm=ones(m.q_lora_rank) if m.q_lora_rank else None,
            q_b=shared(heads * dq, q_in),
            kv_a=shared(m.kv_lora_rank + m.qk_rope_head_dim, cfg.hidden_size, allow_fp8=False),
            kv_a_norm=ones(m.kv_lora_rank),
            w_uk=shared(heads * m.kv_lora_rank, m.qk_nope_head_dim, allow_fp8=False),
            w_uv=shared(heads * m.v_head_dim, m.kv_lora_rank, allow_fp8=False),
            o=shared(cfg.hidden_size, heads * m.v_head_dim))
        if self.device.type == "cuda" and config.get("mla_fold_q"):
            full.q_fold = shared(heads * (m.kv_lora_rank + m.qk_rope_head_dim), q_in)

        def rows(w: LinearWeight, per: int) -> LinearWeight:
            a, b = r * hl * per, (r + 1) * hl * per
            if w.scale is None:
                return LinearWeight(w.weight[a:b])
            assert a % 128 == 0 and b % 128 == 0, "head shard not aligned to the 128-row scale blocks"
            return LinearWeight.from_quantized(w.weight[a:b], w.scale[a // 128:b // 128].contiguous())

        def cols(w: LinearWeight, per: int) -> LinearWeight:
            a, b = r * hl * per, (r + 1) * hl * per
            if w.scale is None:
                return LinearWeight(w.weight[:, a:b].contiguous())
            assert a % 128 == 0 and b % 128 == 0, "head shard not aligned to the 128-column scale blocks"
            return LinearWeight.from_quantized(w.weight[:, a:b].contiguous(), w.scale[:, a // 128:b // 128].contiguous())

        shard = MlaWeights(q_a=full.q_a, q_a_norm=full.q_a_norm, q_b=rows(full.q_b, dq), kv_a=full.kv_a,
                           kv_a_norm=full.kv_a_norm, w_uk=rows(full.w_uk, m.kv_lora_rank),
                           w_uv=rows(full.w_uv, m.v_head_dim), o=cols(full.o, m.v_head_dim),
                           q_fold=None if full.q_fold is None else rows(full.q_fold, m.kv_lora_rank + m.qk_rope_head_dim))
        self._attn_dp_pending = MlaAttention(cfg, full, heads)
        self._attn_dp_pending.reduce_output = False
        return MlaAttention(cfg, shard, hl)

    def weight_bytes(self) -> int:
        n = self.embed.numel() * 2 + self.final_norm.numel() * 2
        if self.lm_head.weight.data_ptr() != self.embed.data_ptr():
            n += self.lm_head.nbytes()
        for lw in self.layers:
            for w in (lw.qkv, lw.o, lw.gate_up, lw.down):
                if w is not None:
                    n += w.nbytes()
            if lw.cross is not None:
                n += lw.cross.nbytes()
            if lw.ffn_module is not None and hasattr(lw.ffn_module, "nbytes"):
                n += lw.ffn_module.nbytes()
            if lw.attn_module is not None and hasattr(lw.attn_module, "nbytes"):
                n += lw.attn_module.nbytes()
            if lw.attn_dp is not None:      # the all-head copy (its head shard above may share storage with it)
                n += lw.attn_dp.nbytes()
        return n

    # ------------------------------------------------------------------------------ KV cache
    def kv_bytes_per_page(self, page: int) -> int:
        if self.cfg.mla is not None:
            return (self.layer1 - self.layer0) * page * (self.cfg.mla.kv_lora_rank + self.cfg.mla.qk_rope_head_dim) * 2
        return (self.layer1 - self.layer0) * 2 * self.hkv * page * self.cfg.head_dim * 2

    def alloc_kv(self, num_pages: int, page: int = 16) -> torch.Tensor:
        """[layers, 2, pages, hkv_local, page, head_dim] bf16, or with multi-head latent attention
        [layers, pages, page, 576] (latent + rotated shared key, replicated on every rank)."""
        if self.cfg.mla is not None:
            row = self.cfg.mla.kv_lora_rank + self.cfg.mla.qk_rope_head_dim
            self.kv_cache = torch.zeros(self.layer1 - self.layer0, num_pages, page, row, dtype=torch.bfloat16,
                                        device=self.device)
            return self.kv_cache
        self.kv_cache = torch.zeros(self.layer1 - self.layer0, 2, num_pages, self.hkv, page, self.cfg.head_dim,
                                    dtype=torch.bfloat16, device=self.device)
        return self.kv_cache

    # ------------------------------------------------------------------------------ forward
    def _attn_scale(self) -> float:
        s = self.cfg.attn_scale if self.cfg.attn_scale > 0 else 1.0 / math.sqrt(self.cfg.head_dim)
        return s * self.rope_attn_factor * self.rope_attn_factor if self.rope_attn_factor != 1.0 else s

    def _reduce_linear(self, x, w: LinearWeight) -> torch.Tensor:
        """Row-parallel linear: local partial product, then sum over the TP group. In order of
        preference: the fused GEMM + all-reduce kernel (up to 128 tokens), GEMM written straight
        into the peer-memory all-reduce kernel's input buffer, GEMM + NCCL."""
        if self.tp > 1:
            m = (x.data if isinstance(x, ops.Fp8Act) else x).shape[0]
            n = w.out_features
            if self.fused_rp is not None and self.fused_rp.supports(m, n) and x_is_cuda(x):
                return self.fused_rp(x, w)[0]
            if self.fused_rp is not None and self.fused_rp.supports_large(m, n) and x_is_cuda(x):
                # prefill chunks: the same kernel in its large-token form (the view is consumed by the
                # residual add that follows, long before its output slot comes round again)
                return self.fused_rp.large(x, w)
            if self.row_parallel_linear is not None and self.fused_rp is None:
                return self.row_parallel_linear(x, w)
            if self.custom_ar is not None and self.custom_ar.fits(m * n):
                ops.linear(x, w, out=self.custom_ar.input(m, n))
                return self.custom_ar.reduce(m, n)
        y = ops.linear(x, w)
        return self.all_reduce(y) if self.tp > 1 else y

    # ------------------------------------------------------------------------------ layer pieces
    def _attention(self, lw: LayerWeights, li: int, h: torch.Tensor, hq8, batch: ForwardBatch, scale: float) -> torch.Tensor:
        """qkv projection, (q/k norm,) rotary + KV-cache write, paged attention, output projection."""
        if lw.attn_module is not None:
            return lw.attn_module(h, batch, li, self)
        return self._reduce_linear(self._attention_core(lw, li, h, hq8, batch, scale), lw.o)

    def _attention_core(self, lw: LayerWeights, li: int, h: Optional[torch.Tensor], hq8, batch: ForwardBatch,
                        scale: float) -> torch.Tensor:
        """Everything of the attention block before the output projection: [T, local heads * d]
        (bf16, or already quantised for an fp8 output projection at decode)."""
        cfg, d = self.cfg, self.cfg.head_dim
        t = (h if h is not None else hq8.data).shape[0]
        # decode-size batches: a fully K-split qkv GEMM leaves its ranges to the rotary kernel
        simple = (not cfg.qk_norm_full and not cfg.qk_norm_after_rope and not (cfg.mrope_section and batch.positions3 is not None)
                  and self.kv_cache is not None)
        qkv = ops.linear(hq8 if hq8 is not None else h, lw.qkv, defer=simple and t <= 128 and x_is_cuda(hq8 if hq8 is not None else h))
        q_norm_w, k_norm_w = lw.q_norm, lw.k_norm
        if cfg.qk_norm_full and q_norm_w is not None:
            # RMSNorm over all heads of q (and of k) at once, before the heads are split
            nq, nk = self.hq * d, self.hkv * d
            qn, _, _ = ops.norm(qkv[:, :nq].contiguous(), q_norm_w, eps=cfg.rms_eps)
            kn, _, _ = ops.norm(qkv[:, nq:nq + nk].contiguous(), k_norm_w, eps=cfg.rms_eps)
            qkv = torch.cat([qn, kn, qkv[:, nq + nk:]], 1)
            q_norm_w = k_norm_w = None
        kc, vc = (self.kv_cache[li, 0], self.kv_cache[li, 1]) if self.kv_cache is not None else (None, None)
        window = cfg.layer_window(self.layer0 + li)
        inv_freq = self.inv_freq_local if (window > 0 and self.inv_freq_local is not None) else self.inv_freq
        rot = cfg.rotary_dim if cfg.use_rope and not (cfg.nope_global and window == 0) else 0
        if cfg.rope_layers and not cfg.rope_layers[self.layer0 + li]:
            rot = 0
        if cfg.mrope_section and batch.positions3 is not None and rot > 0:
            qkv = self._mrope(qkv, batch.positions3, inv_freq)       # rotated here; the kernel below only writes the cache
            rot = 0
        if cfg.qk_norm_after_rope and q_norm_w is not None:
            # rotate first (no cache write), normalise the rotated heads, then run the same kernel with
            # no rotation for the cache write
            qr, kr, vr = ops.rope_kv(qkv, batch.positions, self.hq, self.hkv, d, rot=rot, theta=cfg.rope_theta,
                                     inv_freq=inv_freq, style=cfg.rope_style, want_kv=True)
            qn, _, _ = ops.norm(qr.reshape(-1, d), q_norm_w, eps=cfg.rms_eps)
            kn, _, _ = ops.norm(kr.reshape(-1, d), k_norm_w, eps=cfg.rms_eps)
            qkv = torch.cat([qn.reshape(t, -1), kn.reshape(t, -1), vr.reshape(t, -1)], 1).contiguous()
            q_norm_w = k_norm_w = None
            rot = 0
        q, _, _ = ops.rope_kv(qkv, batch.positions, self.hq, self.hkv, d, k_cache=kc, v_cache=vc,
                              slot_mapping=batch.slot_mapping, rot=rot, theta=cfg.rope_theta,
                              inv_freq=inv_freq, style=cfg.rope_style, q_norm_w=q_norm_w,
                              k_norm_w=k_norm_w, eps=cfg.rms_eps)
        if self.alibi_slopes is not None or lw.sinks is not None:
            att = ops.attn_paged_biased(q, kc, vc, batch.block_table, batch.kv_lens,
                                        None if batch.is_decode else batch.cu_q, scale=scale,
                                        softcap=cfg.attn_softcap, window=window, alibi=self.alibi_slopes,
                                        sinks=lw.sinks)
        elif batch.is_decode:
            if self.fp8 and q.is_cuda and lw.o is not None and lw.o.is_fp8 and d == 128:
                # the split-combine kernel emits the o-projection's fp8 input itself
                _, att8 = ops.attn_decode(q, kc, vc, batch.block_table, batch.kv_lens, scale=scale,
                                          softcap=cfg.attn_softcap, window=window,
                                          max_kv_len=batch.max_kv_len or None, emit_fp8=True, emit_bf16=False)
                return att8
            att = ops.attn_decode(q, kc, vc, batch.block_table, batch.kv_lens, scale=scale,
                                  softcap=cfg.attn_softcap, window=window,
                                  max_kv_len=batch.max_kv_len or None)
        else:
            att = ops.attn_prefill_paged(q, kc, vc, batch.block_table, batch.kv_lens, batch.cu_q,
                                         batch.max_q_len, causal=True, scale=scale,
                                         softcap=cfg.attn_softcap, window=window)
        return att.reshape(t, self.hq * d)

    def _mrope(self, qkv: torch.Tensor, positions3: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
        """Rotary embedding whose frequency pairs are split into three sections, driven by the time,
        row and column position of each token (split-half pairing). Rotates q and k inside the
        packed [T, (hq + 2 hkv) d] activation."""
        cfg, d = self.cfg, self.cfg.head_dim
        t = qkv.shape[0]
        if cfg.mrope_interleaved:         # pair j follows axis j % 3 while that axis has pairs left, else time
            j = torch.arange(d // 2, device=qkv.device)
            lim = torch.tensor([0, cfg.mrope_section[1] * 3, cfg.mrope_section[2] * 3], device=qkv.device)
            axis = torch.where(j < lim[j % 3], j % 3, torch.zeros_like(j))
        else:
            axis = torch.repeat_interleave(torch.arange(3, device=qkv.device),
                                           torch.tensor(cfg.mrope_section, device=qkv.device))      # [d / 2]
        ang = positions3.to(qkv.device).float()[:, :, None] * inv_freq.float()[None, None, :]        # [3, T, d / 2]
        ang = ang.gather(0, axis[None, None, :].expand(1, t, -1))[0]                                 # [T, d / 2]
        cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
        x = qkv.float().reshape(t, self.hq + 2 * self.hkv, d)
        nr = self.hq + self.hkv
        x1, x2 = x[:, :nr, : d // 2], x[:, :nr, d // 2:]
        rotd = torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1)
        return torch.cat([rotd, x[:, nr:]], 1).reshape(t, -1).to(qkv.dtype).contiguous()

    def _block_norm(self, x: torch.Tensor, w: Optional[torch.Tensor], b: Optional[torch.Tensor]) -> torch.Tensor:
        cfg = self.cfg
        return ops.norm(x, w, bias=b, eps=cfg.rms_eps, layernorm=cfg.norm_type == "layernorm",
                        weight_plus_one=cfg.norm_plus_one)[0]

    @staticmethod
    def _activation(x: torch.Tensor, name: str, params: Optional[tuple] = None) -> torch.Tensor:
        xf = x.float()
        if name == "xielu":
            # x > 0: alpha_p x^2 + beta x; otherwise alpha_n (expm1(min(x, eps)) - x) + beta x
            ap, an, beta, eps = params
            y = torch.where(xf > 0, ap * xf * xf + beta * xf,
                            (torch.expm1(torch.clamp(xf, max=eps)) - xf) * an + beta * xf)
        elif name == "silu":
            y = torch.nn.functional.silu(xf)
        elif name == "gelu":
            y = torch.nn.functional.gelu(xf)
        elif name == "gelu_tanh":
            y = torch.nn.functional.gelu(xf, approximate="tanh")
        elif name == "relu2":
            y = torch.relu(xf) ** 2
        elif name == "relu":
            y = torch.relu(xf)
        else:
            raise ValueError(f"unknown activation '{name}'")
        return y.to(x.dtype)

    def _ffn(self, lw: LayerWeights, h: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        if lw.ffn_module is not None:
            return lw.ffn_module(h, self)
        gu = ops.linear(h, lw.gate_up)
        if not cfg.gated_ffn:
            return self._reduce_linear(self._activation(gu, cfg.activation, lw.act_params), lw.down)
        if cfg.activation in ("silu", "gelu_tanh"):
            act, _ = ops.glu(gu, cfg.activation)
        else:
            f = gu.shape[1] // 2
            act = (self._activation(gu[:, :f], cfg.activation, lw.act_params).float() * gu[:, f:].float()).to(gu.dtype)
        return self._reduce_linear(act.contiguous(), lw.down)

    @staticmethod
    def _cross_layer(cross, x: torch.Tensor, batch: ForwardBatch) -> torch.Tensor:
        """A cross-attention layer over each sequence's own vision states (sequences without an image
        pass through unchanged)."""
        cs, rm = batch.cross_states, batch.cross_row_mask
        if cs is None or isinstance(cs, torch.Tensor):
            return cross(x, cs, rm)
        bounds = list(range(len(cs) + 1)) if batch.is_decode or batch.cu_q is None else batch.cu_q.tolist()
        out = x
        for i, st in enumerate(cs):
            if st is None:
                continue
            if out is x:
                out = x.clone()
            a, b = bounds[i], bounds[i + 1]
            out[a:b] = cross(x[a:b], st, None if rm is None else rm[a:b])
        return out

    def _forward_general(self, batch: ForwardBatch, x: torch.Tensor, scale: float):
        """Layer loop for block structures outside the fused path: norms after the blocks instead of
        before (OLMo 2), LayerNorm with bias, parallel attention / feed-forward branches, linear
        biases, non-gated or other activations. ``x`` is the residual stream itself; the kernels
        underneath (GEMMs, rotary + cache write, paged attention) are the same."""
        cfg = self.cfg
        rm = cfg.residual_multiplier

        def add(stream, *deltas):
            y = stream.float()
            for dlt in deltas:
                y = y + (dlt.float() * rm if rm != 1.0 else dlt.float())
            return y.to(stream.dtype)

        for li, lw in enumerate(self.layers):
            if lw.cross is not None:
                x = self._cross_layer(lw.cross, x, batch)
                continue
            h = self._block_norm(x, lw.in_norm, lw.in_norm_b) if cfg.pre_norm else x
            a = self._attention(lw, li, h, None, batch, scale)
            if lw.post_attn_norm is not None:
                a = self._block_norm(a, lw.post_attn_norm, None)
            if cfg.parallel_residual:
                h2 = h if cfg.shared_parallel_norm else self._block_norm(x, lw.post_norm, lw.post_norm_b)
                x = add(x, a, self._ffn(lw, h2))
                continue
            x = add(x, a)
            h2 = self._block_norm(x, lw.post_norm, lw.post_norm_b) if (cfg.pre_norm and lw.post_norm is not None) else x
            f = self._ffn(lw, h2)
            if lw.post_ffn_norm is not None:
                f = self._block_norm(f, lw.post_ffn_norm, None)
            x = add(x, f)
            if batch.deepstack is not None and self.layer0 + li < batch.deepstack.shape[0]:
                x = (x.float() + batch.deepstack[self.layer0 + li].float()).to(x.dtype)
        if not self.last_stage:
            return x, None
        return self._block_norm(x, self.final_norm, self.final_norm_b)

    def _fused_tp_ok(self, tokens: int) -> bool:
        """True when the layer loop can run on the fused row-parallel kernel: a plain pre-norm
        RMSNorm decoder with dense gated feed-forward blocks, held completely by this instance."""
        cfg, frp = self.cfg, self.fused_rp
        if frp is None or self.tp <= 1 or not (self.first_stage and self.last_stage):
            return False
        if not frp.supports(tokens, cfg.hidden_size) or cfg.general_path or not cfg.gated_ffn:
            return False
        if cfg.residual_multiplier != 1.0 or cfg.post_norms or cfg.activation not in ("silu", "gelu_tanh"):
            return False
        return all(lw.qkv is not None and lw.o is not None and lw.gate_up is not None and lw.down is not None
                   and lw.o.bias is None and lw.down.bias is None and lw.post_attn_norm is None
                   and lw.post_ffn_norm is None and lw.cross is None for lw in self.layers)

    def _forward_fused_tp(self, batch: ForwardBatch, x: torch.Tensor) -> torch.Tensor:
        """Layer loop of a tensor-parallel rank for at most 128 tokens. Per layer:

            qkv GEMM -> rope + KV write -> attention -> o GEMM    [all-reduce + residual + norm + fp8 emit]
            gate|up GEMM -> GLU (fp8 emit) -> down GEMM           [all-reduce + residual + norm + fp8 emit]

        where each bracket is the epilogue of the GEMM before it (one kernel), and the second
        bracket already applies the NEXT layer's input norm (the final norm after the last layer).
        The residual stream ``res`` is sharded by token row: each rank keeps only the rows it owns
        up to date, the kernel updates them in place."""
        cfg, frp = self.cfg, self.fused_rp
        fp8 = self.fp8
        scale = self._attn_scale()
        kw = dict(eps=cfg.rms_eps, weight_plus_one=cfg.norm_plus_one)
        lw0 = self.layers[0]
        q8 = fp8 and lw0.qkv.is_fp8
        h, _, hq8 = ops.norm(x, lw0.in_norm, emit_fp8=q8, emit_bf16=not q8, **kw)
        res = x.clone() if batch.embeds is not None else x
        last = len(self.layers) - 1
        for li, lw in enumerate(self.layers):
            att = self._attention_core(lw, li, h, hq8, batch, scale)
            g8 = fp8 and lw.gate_up.is_fp8
            h2, h2q8 = frp(att, lw.o, res=res, norm_w=lw.post_norm, emit_fp8=g8, emit_bf16=not g8, **kw)
            gu = ops.linear(h2q8 if h2q8 is not None else h2, lw.gate_up, defer=True)
            d8 = fp8 and lw.down.is_fp8
            act, act8 = ops.glu(gu, cfg.activation, emit_fp8=d8, emit_bf16=not d8)
            if li == last:
                h, hq8 = frp(act8 if act8 is not None else act, lw.down, res=res, norm_w=self.final_norm, **kw)
            else:
                n8 = fp8 and self.layers[li + 1].qkv.is_fp8
                h, hq8 = frp(act8 if act8 is not None else act, lw.down, res=res,
                             norm_w=self.layers[li + 1].in_norm, emit_fp8=n8, emit_bf16=not n8, **kw)
        return h

    def _dp_attention_ok(self, batch: ForwardBatch) -> bool:
        """True when this decode step can run in the data-parallel attention layout: a plain pre-norm
        RMSNorm stack whose every layer has the all-head attention weights, and a row count the ranks
        divide."""
        ex, cfg = self.dp_exchange, self.cfg
        if ex is None or not batch.is_decode or batch.embeds is not None or not (self.first_stage and self.last_stage):
            return False
        if cfg.general_path or cfg.post_norms or cfg.residual_multiplier != 1.0 or cfg.norm_plus_one:
            return False
        if self.embed_norm_w is not None or self.pos_embed is not None or batch.deepstack is not None:
            return False
        if not ex.supports(batch.tokens.shape[0]):
            return False
        return all(lw.attn_dp is not None and lw.cross is None for lw in self.layers)

    def _forward_dp_attention(self, batch: ForwardBatch) -> torch.Tensor:
        """Decode step with the requests dealt over the ranks for the attention block and the expert /
        feed-forward block run over all rows with this rank's weight shards. Per layer:

            attention of the L local rows (all heads)     [residual + RMSNorm -> every rank's buffer]
            router, experts, shared expert over T rows    [combine -> owning rank; sum + residual + RMSNorm]

        where each bracket is one exchange step (parallel/dp_attention.py). Returns the final-normed
        hidden states of all T rows (one all-gather at the end), like the tensor-parallel path."""
        cfg, ex = self.cfg, self.dp_exchange
        t = batch.tokens.shape[0]
        l = t // self.tp
        sl = slice(self.tp_rank * l, (self.tp_rank + 1) * l)
        lb = ForwardBatch(tokens=batch.tokens[sl], positions=batch.positions[sl], slot_mapping=batch.slot_mapping[sl],
                          block_table=batch.block_table[sl], kv_lens=batch.kv_lens[sl], is_decode=True, max_q_len=1,
                          max_kv_len=batch.max_kv_len)
        res = ops.embedding(lb.tokens, self.embed, cfg.embed_scale * cfg.embedding_multiplier).contiguous()
        h, _, _ = ops.norm(res, self.layers[0].in_norm, eps=cfg.rms_eps)
        fp8 = self.fp8 and res.is_cuda
        last = len(self.layers) - 1
        for li, lw in enumerate(self.layers):
            a = lw.attn_dp(h, lb, li, self)
            cache = self.kv_cache[li] if self.kv_cache is not None else None
            g = ex.gather(a.contiguous(), res, lw.post_norm, cfg.rms_eps, cache, lb.slot_mapping, batch.slot_mapping)
            if lw.ffn_module is not None:
                lw.ffn_module.forward_partial(g, ex)
            else:
                gu = ops.linear(g, lw.gate_up)
                d8 = fp8 and lw.down.is_fp8
                act, act8 = ops.glu(gu, cfg.activation, emit_fp8=d8, emit_bf16=not d8)
                ex.scatter(None, None, None, ops.linear(act8 if act8 is not None else act, lw.down), 0)
            h = ex.reduce(res, self.final_norm if li == last else self.layers[li + 1].in_norm, cfg.rms_eps)
        return self.comm.all_gather(h.contiguous(), dim=0)

    def forward_hidden(self, batch: ForwardBatch, hidden_in: Optional[tuple] = None):
        """Runs this instance's layers. The last pipeline stage (the only one by default) returns the
        final-normed hidden states [T, H]; an earlier stage returns ``(x, residual)`` for the next
        stage, which receives it as ``hidden_in``."""
        cfg = self.cfg
        d = cfg.head_dim
        res: Optional[torch.Tensor] = None
        if hidden_in is None and self._dp_attention_ok(batch):
            return self._forward_dp_attention(batch)
        if hidden_in is not None:
            x, res = hidden_in
        elif batch.embeds is not None:
            x = batch.embeds
        else:
            x = ops.embedding(batch.tokens, self.embed, cfg.embed_scale * cfg.embedding_multiplier)
        if self.embed_norm_w is not None and hidden_in is None:
            x = self._block_norm(x, self.embed_norm_w, self.embed_norm_b)
        if self.pos_embed is not None and hidden_in is None:
            x = (x.float() + self.pos_embed[batch.positions.long() + cfg.learned_position_offset].float()).to(x.dtype)
        scale = self._attn_scale()
        fp8 = self.fp8 and x.is_cuda
        if cfg.general_path:
            return self._forward_general(batch, x if res is None else (x.float() + res.float()).to(x.dtype), scale)
        if hidden_in is None and x.is_cuda and self._fused_tp_ok(x.shape[0]):
            return self._forward_fused_tp(batch, x)

        for li, lw in enumerate(self.layers):
            # ---- attention block
            if res is None:
                h, _, hq8 = ops.norm(x, lw.in_norm, eps=cfg.rms_eps, weight_plus_one=cfg.norm_plus_one,
                                     emit_fp8=fp8 and lw.qkv is not None and lw.qkv.is_fp8, emit_bf16=True)
                res = x
            else:
                h, res, hq8 = ops.norm(x, lw.in_norm, residual=res, eps=cfg.rms_eps,
                                       weight_plus_one=cfg.norm_plus_one,
                                       emit_fp8=fp8 and lw.qkv is not None and lw.qkv.is_fp8, emit_bf16=True)
            a = self._attention(lw, li, h, hq8, batch, scale)
            if lw.post_attn_norm is not None:
                a, _, _ = ops.norm(a, lw.post_attn_norm, eps=cfg.rms_eps, weight_plus_one=cfg.norm_plus_one)
            if cfg.residual_multiplier != 1.0:
                a = (a.float() * cfg.residual_multiplier).to(a.dtype)
            # ---- feed-forward block
            dense_fp8 = fp8 and lw.gate_up is not None and lw.gate_up.is_fp8
            h2, res, h2q8 = ops.norm(a, lw.post_norm, residual=res, eps=cfg.rms_eps,
                                     weight_plus_one=cfg.norm_plus_one, emit_fp8=dense_fp8, emit_bf16=True)
            if lw.ffn_module is not None:
                f = lw.ffn_module(h2, self)
            else:
                gated_fast = cfg.gated_ffn and cfg.activation in ("silu", "gelu_tanh")
                gu = ops.linear(h2q8 if h2q8 is not None else h2, lw.gate_up,
                                defer=gated_fast and x.is_cuda and x.shape[0] <= 128)
                if cfg.gated_ffn:
                    act, act8 = ops.glu(gu, cfg.activation, emit_fp8=fp8 and lw.down.is_fp8,
                                        emit_bf16=not (fp8 and lw.down.is_fp8))
                    f = self._reduce_linear(act8 if act8 is not None else act, lw.down)
                else:
                    f = self._reduce_linear(gu, lw.down)
            if lw.post_ffn_norm is not None:
                f, _, _ = ops.norm(f, lw.post_ffn_norm, eps=cfg.rms_eps, weight_plus_one=cfg.norm_plus_one)
            if cfg.residual_multiplier != 1.0:
                f = (f.float() * cfg.residual_multiplier).to(f.dtype)
            x = f
        if not self.last_stage:
            return x, res
        out, _, _ = ops.norm(x, self.final_norm, residual=res, eps=cfg.rms_eps, weight_plus_one=cfg.norm_plus_one)
        return out

    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        """[rows, H] -> local vocabulary shard logits [rows, vocab_local] (bf16)."""
        y = ops.linear(hidden, self.lm_head)
        cfg = self.cfg
        if cfg.logits_scale != 1.0:
            y = (y.float() * cfg.logits_scale).to(y.dtype)
        if cfg.logit_softcap > 0:
            y = (torch.tanh(y.float() / cfg.logit_softcap) * cfg.logit_softcap).to(y.dtype)
        return y

    def full_logits(self, hidden: torch.Tensor) -> torch.Tensor:
        """Logits over the whole vocabulary (gathers the shards when tensor parallel)."""
        y = self.logits(hidden)
        if self.tp > 1:
            y = self.comm.all_gather(y, dim=1)
        return y[:, : self.cfg.vocab_size]

    def greedy_tokens(self, hidden: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """argmax over the vocabulary; with TP each rank reduces its shard and the (value, index)
        pairs are combined, so only 8 bytes per row and rank cross the wire."""
        y = self.logits(hidden)
        if self.tp == 1:
            if y.shape[1] > self.cfg.vocab_size:
                y = y[:, : self.cfg.vocab_size]
            return ops.argmax(y, out)
        v0 = self.tp_rank * self.vocab_local
        valid = min(self.vocab_local, self.cfg.vocab_size - v0)
        yl = y[:, :valid]
        idx = ops.argmax(yl)
        val = yl.float().gather(1, idx.long()[:, None])[:, 0]
        packed = torch.stack([val, (idx + v0).float()], dim=1)          # [rows, 2]
        allp = self.comm.all_gather(packed.unsqueeze(0), dim=0)         # [tp, rows, 2]
        vals, ids = allp[..., 0], allp[..., 1]
        best = vals.argmax(dim=0)                                       # first max -> lowest rank -> lowest id
        tok = ids.gather(0, best[None])[0].to(torch.int32)
        if out is not None:
            out.copy_(tok)
            return out
        return tok
