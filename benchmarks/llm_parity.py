"""Multi-GPU correctness check that ``bench.py`` runs before its timed region: a two-layer slice of
the benchmarked LLM architecture (same hidden size, heads, feed-forward / expert shapes; smaller
vocabulary) is built once from full weights, sharded over the N ranks exactly as the benchmark
model is, and run on a short prompt; rank 0 also builds the unsharded model from the same weights.
The cosine between the two sets of logits (minimum over rows) and the share of identical greedy
tokens are reported. With fused tensor-parallel kernels enabled, the sharded run goes through them
(the prompt is shorter than their 128-token limit)."""
from __future__ import annotations

import zlib
from dataclasses import replace

import torch

from hartsyinference_b200 import ops
from hartsyinference_b200.models.llm.transformer import DecoderModel, ForwardBatch
from hartsyinference_b200.parallel.comm import SingleComm

PARITY_VOCAB = 16384


def _shape(name: str, cfg) -> tuple:
    H = cfg.hidden_size
    mla, moe = cfg.mla, cfg.moe
    leaf = name.rsplit(".", 2)[-2] if name.endswith(".weight") else name.rsplit(".", 1)[-1]
    if leaf in ("embed_tokens", "lm_head"):
        return (cfg.vocab_size, H)
    if leaf == "q_a_layernorm":
        return (mla.q_lora_rank,)
    if leaf == "kv_a_layernorm":
        return (mla.kv_lora_rank,)
    if "layernorm" in leaf or leaf == "norm":
        return (H,)
    if leaf == "e_score_correction_bias":
        return (moe.num_experts,)
    if leaf == "gate" and ".mlp.gate." in name:
        return (moe.num_experts, H)
    if mla is not None and ".self_attn." in name:
        dq = mla.qk_nope_head_dim + mla.qk_rope_head_dim
        return {"q_a_proj": (mla.q_lora_rank, H), "q_b_proj": (cfg.num_heads * dq, mla.q_lora_rank),
                "q_proj": (cfg.num_heads * dq, H),
                "kv_a_proj_with_mqa": (mla.kv_lora_rank + mla.qk_rope_head_dim, H),
                "kv_b_proj": (cfg.num_heads * (mla.qk_nope_head_dim + mla.v_head_dim), mla.kv_lora_rank),
                "o_proj": (H, cfg.num_heads * mla.v_head_dim)}[leaf]
    if ".self_attn." in name:
        return {"q_proj": (cfg.q_size, H), "k_proj": (cfg.kv_size, H), "v_proj": (cfg.kv_size, H),
                "o_proj": (H, cfg.q_size)}[leaf]
    if ".shared_expert." in name:
        raise KeyError(name)
    if ".experts." in name:
        f = moe.expert_ffn
    elif ".shared_experts." in name:
        f = moe.shared_ffn * moe.num_shared_experts
    else:
        f = cfg.ffn_size
    return {"gate_proj": (f, H), "up_proj": (f, H), "down_proj": (H, f)}[leaf]


def _weights(cfg, dev):
    """``get(name)`` producing each full tensor on the device from a seed derived from its name:
    identical on every rank, never all resident at once."""
    def get(name: str):
        if name.endswith(".bias") and "e_score_correction_bias" not in name:
            return None
        try:
            shape = _shape(name, cfg)
        except KeyError:
            return None
        if len(shape) == 1 and "e_score_correction_bias" not in name:
            return torch.ones(shape, dtype=torch.bfloat16, device=dev)
        t = torch.empty(shape if len(shape) == 2 else (1, shape[0]), dtype=torch.bfloat16, device=dev)
        ops.fill_random_(t, zlib.crc32(name.encode()) + 1, 0.05 if ".mlp.gate." in name else 0.02)
        return t if len(shape) == 2 else t.reshape(-1).float()
    return get


def run(cfg, comm, dev, fp8: bool, enable_fused=None, dp_attention: bool = False, dp_fused=None) -> dict:
    """All ranks call this. ``enable_fused(model)`` (optional) switches the sharded model to the
    fused kernels the benchmark will use. ``dp_attention``: the sharded model also runs one decode step
    of ``2 x ranks`` requests in the data-parallel attention layout (after prefilling them in the
    tensor-parallel layout) and its logits are compared too (``decode_*`` fields)."""
    moe = cfg.moe
    if moe is not None and moe.num_experts > 0:
        moe = replace(moe, first_dense_layers=min(1, moe.first_dense_layers))
    cfg2 = replace(cfg, num_layers=2, vocab_size=PARITY_VOCAB, moe=moe)
    get = _weights(cfg2, dev)
    t = 48
    g = torch.Generator().manual_seed(3)
    toks = torch.randint(0, cfg2.vocab_size, (t,), generator=g).to(torch.int32).to(dev)

    def forward(model):
        model.alloc_kv(8, 16)
        b = ForwardBatch(tokens=toks, positions=torch.arange(t, dtype=torch.int32, device=dev),
                         slot_mapping=torch.arange(t, dtype=torch.int64, device=dev),
                         block_table=torch.arange(8, dtype=torch.int32, device=dev)[None],
                         kv_lens=torch.tensor([t], dtype=torch.int32, device=dev), is_decode=False,
                         cu_q=torch.tensor([0, t], dtype=torch.int32, device=dev), max_q_len=t, max_kv_len=t)
        return model.full_logits(model.forward_hidden(b)).float()

    seqs, plen, page = 2 * comm.world, 24, 32

    def decode_step(model):
        """Prefill ``seqs`` requests of ``plen`` tokens (one page each), then one decode step of all of
        them with fixed input tokens: [seqs, vocab] logits."""
        model.alloc_kv(seqs + 1, page)
        gd = torch.Generator().manual_seed(11)
        tok = torch.randint(0, cfg2.vocab_size, (seqs * plen,), generator=gd).to(torch.int32).to(dev)
        nxt = torch.randint(0, cfg2.vocab_size, (seqs,), generator=gd).to(torch.int32).to(dev)
        ar = torch.arange(seqs, device=dev)
        table = ar.to(torch.int32)[:, None].contiguous()
        b = ForwardBatch(tokens=tok, positions=torch.arange(plen, dtype=torch.int32, device=dev).repeat(seqs),
                         slot_mapping=(ar[:, None] * page + torch.arange(plen, device=dev)[None]).reshape(-1).to(torch.int64),
                         block_table=table, kv_lens=torch.full((seqs,), plen, dtype=torch.int32, device=dev), is_decode=False,
                         cu_q=(torch.arange(seqs + 1, dtype=torch.int32, device=dev) * plen), max_q_len=plen, max_kv_len=plen)
        model.forward_hidden(b)
        b = ForwardBatch(tokens=nxt, positions=torch.full((seqs,), plen, dtype=torch.int32, device=dev),
                         slot_mapping=(ar * page + plen).to(torch.int64), block_table=table,
                         kv_lens=torch.full((seqs,), plen + 1, dtype=torch.int32, device=dev), is_decode=True,
                         max_q_len=1, max_kv_len=plen + 1)
        return model.full_logits(model.forward_hidden(b)).float()

    dp_attention = dp_attention and cfg2.mla is not None and comm.world > 1
    sharded = DecoderModel(cfg2, dev, comm=comm, fp8=fp8, dp_attention=dp_attention)
    sharded.load_state_dict(get)
    path = "nccl"
    if enable_fused is not None and enable_fused(sharded):
        path = "fused"
    got = forward(sharded)
    got_dec, dp_path = None, None
    if dp_attention:
        from hartsyinference_b200.parallel.dp_attention import enable_dp_attention
        dp_path = "fused" if enable_dp_attention(sharded, comm, max_rows=seqs, fused=dp_fused) else "collectives"
        got_dec = decode_step(sharded)
    if dev.type == "cuda":
        torch.cuda.synchronize()
    for name in ("fused_rp", "custom_ar", "dp_exchange"):
        obj = getattr(sharded, name, None)
        if obj is not None:
            obj.close()
    del sharded
    res = torch.zeros(7, device=dev)
    if comm.rank == 0:
        one = DecoderModel(cfg2, dev, comm=SingleComm(), fp8=fp8)
        one.load_state_dict(get)
        ref = forward(one)
        rows = torch.nn.functional.cosine_similarity(got, ref, dim=-1)
        res[0] = rows.min()
        res[1] = (got.argmax(-1) == ref.argmax(-1)).float().mean()
        res[2] = rows.median()
        res[3] = (rows < 0.99).float().sum()
        if got_dec is not None:
            ref_dec = decode_step(one)
            rows = torch.nn.functional.cosine_similarity(got_dec, ref_dec, dim=-1)
            res[4], res[5] = rows.min(), rows.median()
            res[6] = (got_dec.argmax(-1) == ref_dec.argmax(-1)).float().mean()
        del one
    comm.broadcast(res, 0)
    if dev.type == "cuda":
        torch.cuda.empty_cache()
    cos, agree, med, low, dcos, dmed, dagree = (float(v) for v in res.tolist())
    out = {"ok": cos > 0.99, "cos": cos, "cos_median": med, "rows_below_0.99": int(low), "greedy_agreement": agree, "path": path,
           "what": f"2-layer slice (vocab {PARITY_VOCAB}), {t}-token prompt, {comm.world} ranks vs 1; cos = minimum over rows"}
    if cfg.moe is not None and cfg.moe.num_experts > 0:
        # random-init routers put many tokens on near-ties between experts; the sharded run sums in another
        # order, so a few rows pick a different expert set and differ as a whole, the others agree closely
        out["ok"] = med > 0.99 and cos > 0.9
        out["what"] += "; MoE: rows whose near-tied routing flips differ, judged by the median row (and minimum > 0.9)"
    if dp_path is not None:
        out.update(decode_cos=dcos, decode_cos_median=dmed, decode_greedy_agreement=dagree, decode_path=dp_path,
                   decode_what=f"one decode step of {seqs} requests after a {plen}-token prefill, attention data parallel")
        out["ok"] = bool(out["ok"] and dmed > 0.99 and dcos > 0.9)
    return out
