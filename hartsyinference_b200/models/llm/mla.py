"""Multi-head latent attention (DeepSeek-V2 / V3) on a paged latent cache.

Per token the cache holds the normalised 512-wide latent plus the 64 rotated shared-key values
(576 bf16), not per-head keys and values. Queries are absorbed through ``W_uk`` so attention is
multi-query over latent rows, and ``W_uv`` is applied to the 512-wide result; the o-projection is
row-parallel over heads (one all-reduce, or the fused GEMM + all-reduce hook of the model).

Call sequence on the device (all custom kernels, CUDA-graph capturable in decode):
q_a GEMM -> RMSNorm -> q_b GEMM | kv_a GEMM -> ``mla_prep`` (latent norm, RoPE, cache write, q_pe
RoPE) -> column-batched GEMM (absorb) -> ``mla_attn`` -> column-batched GEMM (W_uv) -> o GEMM.

Reference behaviour: src/HartsyInference.LLM/Transformer/MlaAttention.cs (expands K and V for
every head and attends over a contiguous cache); Hugging Face ``DeepseekV3Attention`` for the
tensor naming (q_a_proj, q_a_layernorm, q_b_proj, kv_a_proj_with_mqa, kv_a_layernorm, kv_b_proj).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

from ... import ops
from ...ops import LinearWeight
from .config import TransformerConfig

LATENT, ROPE, ROW = ops.core.MLA_LATENT, ops.core.MLA_ROPE, ops.core.MLA_ROW


@dataclass
class MlaWeights:
    q_a: Optional[LinearWeight]          # [q_lora, H] (None: q_b maps the hidden state directly)
    q_a_norm: Optional[torch.Tensor]     # [q_lora]
    q_b: LinearWeight                    # [heads_local * (nope + rope), q_lora or H]
    kv_a: LinearWeight                   # [512 + 64, H]   (replicated on every rank)
    kv_a_norm: torch.Tensor              # [512]
    w_uk: LinearWeight                   # stacked [heads_local * 512, nope]: W_uk[h]^T
    w_uv: LinearWeight                   # stacked [heads_local * v_dim, 512]
    o: LinearWeight                      # [H, heads_local * v_dim]
    # optional: q_b with W_uk folded in, [heads_local * 576, q_lora or H]; per head 512 rows
    # W_uk[h]^T W_qb_nope[h] followed by the 64 rotary rows of q_b. Small batches then get the absorbed
    # query from ONE weight-streaming GEMM instead of q_b plus a per-head projection with K = 128.
    q_fold: Optional[LinearWeight] = None

    def all(self):
        return [w for w in (self.q_a, self.q_b, self.kv_a, self.w_uk, self.w_uv, self.o, self.q_fold) if w is not None]


FOLD_MAX_TOKENS = 256      # above this the extra rows of the folded projection cost more than they save


def fold_q(q_b: torch.Tensor, w_uk: torch.Tensor, heads: int, nope: int, rope: int) -> torch.Tensor:
    """``q_b`` [heads * (nope + rope), K] and the stacked ``w_uk`` [heads * 512, nope] -> the folded
    projection [heads * 576, K] (fp32 product, returned in q_b's dtype)."""
    k = q_b.shape[1]
    qb = q_b.float().reshape(heads, nope + rope, k)
    uk = w_uk.float().reshape(heads, -1, nope)
    top = torch.bmm(uk, qb[:, :nope])                              # [heads, 512, K]
    return torch.cat([top, qb[:, nope:]], dim=1).reshape(heads * (uk.shape[1] + rope), k).to(q_b.dtype)


def split_kv_b(kv_b: torch.Tensor, heads: int, nope: int, v_dim: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Split a Hugging Face ``kv_b_proj.weight`` [heads * (nope + v), 512] into the stacked absorbed
    forms: ``w_uk`` [heads * 512, nope] (per head the transpose of its key rows) and ``w_uv``
    [heads * v, 512]."""
    w = kv_b.reshape(heads, nope + v_dim, -1)
    w_uk = w[:, :nope, :].transpose(1, 2).contiguous().reshape(heads * w.shape[2], nope)
    w_uv = w[:, nope:, :].contiguous().reshape(heads * v_dim, w.shape[2])
    return w_uk, w_uv


class MlaAttention:
    """Callable ``(h [T, H], batch, layer_index, model) -> [T, H]`` for ``LayerWeights.attn_module``."""

    def __init__(self, cfg: TransformerConfig, weights: MlaWeights, heads_local: int):
        m = cfg.mla
        assert m is not None and m.kv_lora_rank == LATENT and m.qk_rope_head_dim == ROPE, \
            "the latent kernels are built for kv_lora_rank 512 and 64 rotary dims"
        self.cfg, self.m, self.w = cfg, m, weights
        self.heads = heads_local
        self.dq = m.qk_nope_head_dim + m.qk_rope_head_dim
        # False: the output projection covers all heads on this rank (data-parallel attention), so there
        # is nothing to sum over the ranks
        self.reduce_output = True

    def nbytes(self) -> int:
        n = sum(w.nbytes() for w in self.w.all())
        return n + self.w.kv_a_norm.numel() * 2 + (self.w.q_a_norm.numel() * 2 if self.w.q_a_norm is not None else 0)

    def scale(self, model) -> float:
        s = self.m.attn_scale if self.m.attn_scale > 0 else 1.0 / math.sqrt(self.dq)
        f = getattr(model, "rope_attn_factor", 1.0)
        return s * f * f

    @staticmethod
    def row_lengths(batch, t: int, device) -> tuple[Optional[torch.Tensor], torch.Tensor]:
        """(row -> block-table row or None, row -> causal kv length)."""
        if batch.is_decode:
            return None, batch.kv_lens
        cu = batch.cu_q.to(torch.int64)
        rows = torch.arange(t, device=device, dtype=torch.int64)
        seq = torch.bucketize(rows, cu[1:], right=True)
        seq = seq.clamp_(max=cu.numel() - 2)
        last = cu[1:][seq] - 1
        lens = batch.kv_lens.to(torch.int64)[seq] - (last - rows)
        return seq.to(torch.int32), lens.clamp_(min=0).to(torch.int32)

    def __call__(self, h: torch.Tensor, batch, li: int, model) -> torch.Tensor:
        cfg, m, w = self.cfg, self.m, self.w
        t = h.shape[0]
        qin = h
        if w.q_a is not None:
            qa = ops.linear(h, w.q_a)
            qin, _, _ = ops.norm(qa, w.q_a_norm, eps=cfg.rms_eps)
        kv = ops.linear(h, w.kv_a)
        cache = model.kv_cache[li] if model.kv_cache is not None else None      # [pages, page, 576]
        if w.q_fold is not None and t <= FOLD_MAX_TOKENS:
            # absorbed queries straight from the folded projection; the rotary part is rotated in place
            q_abs = ops.linear(qin, w.q_fold).view(t, self.heads, ROW)
            ops.mla_prep(kv, w.kv_a_norm, q_abs.view(t, self.heads * ROW), q_abs, cache, batch.positions,
                         batch.slot_mapping, model.inv_freq, self.heads, ROW, LATENT, eps=cfg.rms_eps)
        else:
            q = ops.linear(qin, w.q_b)
            q_abs = torch.empty(t, self.heads, ROW, dtype=h.dtype, device=h.device)
            ops.mla_prep(kv, w.kv_a_norm, q, q_abs, cache, batch.positions, batch.slot_mapping, model.inv_freq,
                         self.heads, self.dq, m.qk_nope_head_dim, eps=cfg.rms_eps)
            ops.colbatched_linear(q, w.w_uk.weight, self.heads, self.dq, q_abs.view(t, self.heads * ROW), ROW)
        row_seq, row_len = self.row_lengths(batch, t, h.device)
        lat = ops.mla_attn(q_abs, cache, batch.block_table, row_len, self.scale(model), row_seq=row_seq,
                           max_kv_len=batch.max_kv_len or None)
        v = torch.empty(t, self.heads * m.v_head_dim, dtype=h.dtype, device=h.device)
        ops.colbatched_linear(lat.view(t, self.heads * LATENT), w.w_uv.weight, self.heads, LATENT, v, m.v_head_dim)
        return model._reduce_linear(v, w.o) if self.reduce_output else ops.linear(v, w.o)


def mla_reference(h: torch.Tensor, positions: torch.Tensor, cfg: TransformerConfig, full: dict,
                  inv_freq: torch.Tensor, scale: float) -> torch.Tensor:
    """Causal fp32 oracle for ONE sequence starting at position 0, in the expanded (non-absorbed)
    form with Hugging Face tensors: ``q_a`` / ``q_a_norm`` / ``q_b`` (or ``q``), ``kv_a``,
    ``kv_a_norm``, ``kv_b`` [heads * (nope + v), 512], ``o``."""
    from ...ops import reference as R
    m = cfg.mla
    heads = cfg.num_heads
    x = h.float()
    t = x.shape[0]

    def rms(v, w):
        return v * torch.rsqrt((v * v).mean(-1, keepdim=True) + cfg.rms_eps) * w.float()

    if "q_a" in full:
        q = rms(x @ full["q_a"].float().t(), full["q_a_norm"]) @ full["q_b"].float().t()
    else:
        q = x @ full["q"].float().t()
    q = q.reshape(t, heads, m.qk_nope_head_dim + m.qk_rope_head_dim)
    q_nope, q_pe = q[..., :m.qk_nope_head_dim], q[..., m.qk_nope_head_dim:]
    kv = x @ full["kv_a"].float().t()
    c = rms(kv[:, :m.kv_lora_rank], full["kv_a_norm"])
    k_pe = R.apply_rope(kv[:, m.kv_lora_rank:].unsqueeze(1), positions, inv_freq, 1)
    q_pe = R.apply_rope(q_pe, positions, inv_freq, 1)
    kvb = (c @ full["kv_b"].float().t()).reshape(t, heads, m.qk_nope_head_dim + m.v_head_dim)
    k_nope, v = kvb[..., :m.qk_nope_head_dim], kvb[..., m.qk_nope_head_dim:]
    k = torch.cat([k_nope, k_pe.expand(t, heads, -1)], dim=-1)
    qq = torch.cat([q_nope, q_pe], dim=-1)
    sc = torch.einsum("thd,shd->hts", qq, k) * scale
    mask = torch.ones(t, t, dtype=torch.bool).tril()
    sc = sc.masked_fill(~mask, float("-inf"))
    o = torch.einsum("hts,shd->thd", torch.softmax(sc, dim=-1), v).reshape(t, heads * m.v_head_dim)
    return o @ full["o"].float().t()
