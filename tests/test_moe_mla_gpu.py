"""GPU numerics of the MoE and latent-attention kernels against fp32 PyTorch statements."""
import math

import pytest
import torch

from hartsyinference_b200 import ops
from hartsyinference_b200.ops import LinearWeight
from hartsyinference_b200.ops import _native as N
from hartsyinference_b200.ops import reference as R

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel(a, b):
    return (a.float() - b.float()).abs().max().item() / (b.float().abs().max().item() + 1e-9)


@pytest.mark.parametrize("experts,top_k,n_group,topk_group,sigmoid", [
    (8, 2, 1, 1, False), (64, 6, 1, 1, False), (256, 8, 8, 4, True), (128, 8, 1, 1, True), (60, 4, 1, 1, False)])
def test_route_matches_reference(experts, top_k, n_group, topk_group, sigmoid):
    torch.manual_seed(experts)
    lg = torch.randn(37, experts, device=DEV)
    bias = (torch.randn(experts, device=DEV) * 0.1) if sigmoid else None
    ids, w = ops.moe_route(lg, bias, top_k, n_group=n_group, topk_group=topk_group, sigmoid=sigmoid,
                           norm_topk=True, scale=2.5)
    rids, rw = R.moe_route(lg.cpu(), None if bias is None else bias.cpu(), top_k, n_group, topk_group, sigmoid, True, 2.5)
    assert torch.equal(ids.cpu(), rids)
    assert torch.allclose(w.cpu(), rw, atol=1e-5, rtol=1e-4)
    # bf16 logits take the same path
    ids2, _ = ops.moe_route(lg.to(torch.bfloat16), bias, top_k, n_group=n_group, topk_group=topk_group,
                            sigmoid=sigmoid, norm_topk=True, scale=2.5)
    rids2, _ = R.moe_route(lg.to(torch.bfloat16).float().cpu(), None if bias is None else bias.cpu(), top_k,
                           n_group, topk_group, sigmoid, True, 2.5)
    assert torch.equal(ids2.cpu(), rids2)


def test_dispatch_and_combine_roundtrip():
    torch.manual_seed(1)
    t, k, dim, e, e0, el, cap = 23, 4, 256, 16, 4, 8, 32
    x = torch.randn(t, dim, device=DEV).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(e, device=DEV)[:k] for _ in range(t)]).to(torch.int32)
    w = torch.rand(t, k, device=DEV)
    xs = torch.zeros(el * cap, dim, dtype=torch.bfloat16, device=DEV)
    slot_of, counts = ops.moe_dispatch(x, ids, e0, el, cap, xs)
    local = (ids >= e0) & (ids < e0 + el)
    assert torch.equal(slot_of >= 0, local)
    exp_counts = torch.stack([(ids == e0 + j).sum() for j in range(el)]).to(torch.int32)
    assert torch.equal(counts, exp_counts)
    s = slot_of[local].long()
    assert s.unique().numel() == s.numel()                                       # no slot handed out twice
    assert torch.equal(torch.div(s, cap, rounding_mode="floor"), (ids[local] - e0).long())
    tok = torch.arange(t, device=DEV).unsqueeze(1).expand(t, k)[local]
    assert torch.equal(xs[s], x[tok])
    # combine with y = xs: out[t] = sum over local picks of w * x[t]
    out = torch.zeros(t, dim, dtype=torch.bfloat16, device=DEV)
    ops.moe_combine(xs, slot_of, w, out)
    ref = (w * local).sum(1, keepdim=True) * x.float()
    assert _rel(out, ref) < 0.01
    base = torch.randn(t, dim, device=DEV).to(torch.bfloat16)
    out2 = base.clone()
    ops.moe_combine(xs, slot_of, w, out2, accumulate=True)
    assert _rel(out2, ref + base.float()) < 0.01


@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("groups,m,n,k", [(4, 16, 256, 512), (8, 32, 128, 1024), (3, 128, 384, 256), (32, 16, 4096, 7168)])
def test_grouped_gemm_matches_per_group_matmul(fp8, groups, m, n, k):
    torch.manual_seed(groups * m)
    x = (torch.randn(groups * m, k, device=DEV) * 0.5).to(torch.bfloat16)
    w = (torch.randn(groups * n, k, device=DEV) * 0.05).to(torch.bfloat16)
    lw = LinearWeight.from_dense(w, fp8=fp8)
    y = ops.grouped_linear(x, lw, groups)
    if fp8:
        xq = ops.quant_fp8_act(x, tile_rows=m)
        xr = R.dequant_fp8_act(xq.data.cpu(), xq.scales_fp32().cpu())
        wr = R.dequant_fp8_weight(lw.weight.cpu(), lw.scale.cpu())
    else:
        xr, wr = x.float().cpu(), w.float().cpu()
    ref = torch.cat([xr[g * m:(g + 1) * m] @ wr[g * n:(g + 1) * n].t() for g in range(groups)])
    assert _rel(y.cpu(), ref) < 0.01


def test_grouped_gemm_skips_idle_groups():
    groups, m, n, k = 6, 16, 256, 512
    x = torch.randn(groups * m, k, device=DEV).to(torch.bfloat16)
    lw = LinearWeight(torch.randn(groups * n, k, device=DEV).to(torch.bfloat16) * 0.05)
    counts = torch.tensor([3, 0, 16, 0, 1, 0], dtype=torch.int32, device=DEV)
    out = torch.full((groups * m, n), 7.0, dtype=torch.bfloat16, device=DEV)
    ops.grouped_linear(x, lw, groups, counts=counts, out=out)
    full = ops.grouped_linear(x, lw, groups)
    for g in range(groups):
        blk = out[g * m:(g + 1) * m]
        if counts[g] == 0:
            assert torch.all(blk == 7.0)
        else:
            assert torch.equal(blk, full[g * m:(g + 1) * m])


@pytest.mark.parametrize("t", [1, 5, 64, 128, 200])
def test_colbatched_gemm(t):
    torch.manual_seed(t)
    heads, nope, lat = 16, 128, 512
    q = (torch.randn(t, heads * 192, device=DEV) * 0.5).to(torch.bfloat16)
    w_uk = (torch.randn(heads * lat, nope, device=DEV) * 0.05).to(torch.bfloat16)
    out = torch.zeros(t, heads * 576, dtype=torch.bfloat16, device=DEV)
    ops.colbatched_linear(q, w_uk, heads, 192, out, 576)
    ref = torch.zeros(t, heads * 576)
    ops.colbatched_linear(q.cpu(), w_uk.cpu(), heads, 192, ref, 576)
    assert _rel(out.cpu(), ref) < 0.01
    assert torch.all(out.view(t, heads, 576)[:, :, 512:] == 0)        # the rope tail is not touched
    # value projection: K = 512 per head
    latv = (torch.randn(t, heads * lat, device=DEV) * 0.5).to(torch.bfloat16)
    w_uv = (torch.randn(heads * 128, lat, device=DEV) * 0.05).to(torch.bfloat16)
    v = torch.zeros(t, heads * 128, dtype=torch.bfloat16, device=DEV)
    ops.colbatched_linear(latv, w_uv, heads, lat, v, 128)
    vr = torch.zeros(t, heads * 128)
    ops.colbatched_linear(latv.cpu(), w_uv.cpu(), heads, lat, vr, 128)
    assert _rel(v.cpu(), vr) < 0.01


def test_mla_prep_matches_cpu_statement():
    torch.manual_seed(3)
    t, heads, page, pages = 13, 16, 16, 6
    kv = torch.randn(t, 576, device=DEV).to(torch.bfloat16)
    wn = (1 + 0.1 * torch.randn(512, device=DEV)).to(torch.bfloat16)
    q = torch.randn(t, heads * 192, device=DEV).to(torch.bfloat16)
    pos = torch.arange(100, 100 + t, dtype=torch.int32, device=DEV)
    slots = torch.randperm(pages * page, device=DEV)[:t].to(torch.int64)
    slots[3] = -1
    inv = R.rope_inv_freq(64, 10000.0, DEV)
    cache = torch.zeros(pages, page, 576, dtype=torch.bfloat16, device=DEV)
    q_abs = torch.zeros(t, heads, 576, dtype=torch.bfloat16, device=DEV)
    ops.mla_prep(kv, wn, q, q_abs, cache, pos, slots, inv, heads, 192, 128)
    cache_r = torch.zeros(pages, page, 576, dtype=torch.bfloat16)
    q_abs_r = torch.zeros(t, heads, 576, dtype=torch.bfloat16)
    ops.mla_prep(kv.cpu(), wn.cpu(), q.cpu(), q_abs_r, cache_r, pos.cpu(), slots.cpu(), inv.cpu(), heads, 192, 128)
    assert _rel(cache.cpu(), cache_r) < 0.01
    assert _rel(q_abs.cpu(), q_abs_r) < 0.01


@pytest.mark.parametrize("heads,page,splits", [(16, 16, None), (16, 64, 1), (128, 16, 3), (4, 8, 2), (32, 32, 8)])
def test_mla_attention_matches_fp32(heads, page, splits):
    torch.manual_seed(heads + page)
    lens = [1, 63, 64, 65, 300, 1000]
    rows = len(lens)
    max_pages = (max(lens) + page - 1) // page
    pool = rows * max_pages + 1
    cache = (torch.randn(pool, page, 576, device=DEV) * 0.5).to(torch.bfloat16)
    perm = torch.randperm(pool - 1, device=DEV)[:rows * max_pages].to(torch.int32) + 1
    table = perm.reshape(rows, max_pages).contiguous()
    q = (torch.randn(rows, heads, 576, device=DEV) * 0.3).to(torch.bfloat16)
    kv_lens = torch.tensor(lens, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(192)
    out = ops.mla_attn(q, cache, table, kv_lens, scale, splits=splits, max_kv_len=max(lens))
    ref = ops.mla_attn(q.cpu(), cache.cpu(), table.cpu(), kv_lens.cpu(), scale)
    assert _rel(out.cpu(), ref) < 0.02


def test_mla_attention_row_seq_and_empty_rows():
    torch.manual_seed(5)
    heads, page = 16, 16
    cache = (torch.randn(40, page, 576, device=DEV) * 0.5).to(torch.bfloat16)
    table = torch.arange(1, 33, dtype=torch.int32, device=DEV).reshape(2, 16)
    row_seq = torch.tensor([0, 0, 1, 1, 1], dtype=torch.int32, device=DEV)
    kv_lens = torch.tensor([9, 10, 0, 200, 201], dtype=torch.int32, device=DEV)
    q = (torch.randn(5, heads, 576, device=DEV) * 0.3).to(torch.bfloat16)
    out = ops.mla_attn(q, cache, table, kv_lens, 0.07, row_seq=row_seq, splits=2)
    ref = ops.mla_attn(q.cpu(), cache.cpu(), table.cpu(), kv_lens.cpu(), 0.07, row_seq=row_seq.cpu())
    assert torch.all(out[2] == 0)
    assert _rel(out.cpu(), ref) < 0.02


def test_toy_deepseek_gpu_matches_cpu_model():
    from dataclasses import replace
    from hartsyinference_b200.engine import LLMEngine, SamplingParams
    from hartsyinference_b200.models.llm import config as C
    from hartsyinference_b200.models.llm.transformer import DecoderModel
    moe = C.MoeConfig(num_experts=16, top_k=4, expert_ffn=128, num_shared_experts=1, shared_ffn=128,
                      scoring="sigmoid", norm_topk_prob=True, routed_scaling_factor=2.5, n_group=4,
                      topk_group=2, use_correction_bias=True, first_dense_layers=1)
    mla = C.MlaConfig(q_lora_rank=128, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128)
    cfg = C.tiny("deepseek-v3", hidden_size=256, num_heads=16, num_kv_heads=16, head_dim=192, moe=moe, mla=mla,
                 num_layers=3)
    for fp8 in (False, True):
        model = DecoderModel(cfg, DEV, fp8=fp8)
        model.random_init(0, std=0.05)
        eng = LLMEngine(model, num_pages=64, page_size=16, max_batch=8, prefill_chunk=64, max_model_len=256)
        prompts = [[5, 6, 7, 8, 9, 10, 11], list(range(20, 60))]
        a = eng.generate(prompts, SamplingParams(greedy=True, max_tokens=8))
        b = eng.generate(prompts, SamplingParams(greedy=True, max_tokens=8))
        assert a == b and all(len(x) == 8 for x in a)
        assert eng.model.kv_cache.shape[-1] == 576


def test_dispatch_and_grouped_gemm_with_several_runs_per_expert():
    torch.manual_seed(9)
    t, k, dim, e_local, n = 300, 4, 256, 6, 256
    chunks, cap = 3, 128
    x = torch.randn(t, dim, device=DEV).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(e_local, device=DEV)[:k] for _ in range(t)]).to(torch.int32)
    xs = torch.zeros(e_local * chunks * cap, dim, dtype=torch.bfloat16, device=DEV)
    slot_of, counts = ops.moe_dispatch(x, ids, 0, e_local, cap, xs, chunks=chunks)
    assert counts.numel() == e_local * chunks and int(counts.sum()) == t * k
    blk = torch.div(slot_of.long(), cap, rounding_mode="floor")
    tok_run = (torch.arange(t, device=DEV) // 128)[:, None].expand(t, k)
    assert torch.equal(blk, ids.long() * chunks + tok_run)                 # block = expert * runs + run of the token
    tok = torch.arange(t, device=DEV)[:, None].expand(t, k)
    assert torch.equal(xs[slot_of.long().flatten()], x[tok.flatten()])
    for fp8 in (False, True):
        w = (torch.randn(e_local * n, dim, device=DEV) * 0.05).to(torch.bfloat16)
        lw = LinearWeight.from_dense(w, fp8=fp8)
        y = ops.grouped_linear(xs, lw, e_local, counts=counts, chunks=chunks)
        wr = R.dequant_fp8_weight(lw.weight.cpu(), lw.scale.cpu()) if fp8 else w.float().cpu()
        if fp8:
            xq = ops.quant_fp8_act(xs, tile_rows=cap)
            xr = R.dequant_fp8_act(xq.data.cpu(), xq.scales_fp32().cpu())
        else:
            xr = xs.float().cpu()
        for b in range(e_local * chunks):
            if int(counts[b]) == 0:
                continue
            e = b // chunks
            ref = xr[b * cap:(b + 1) * cap] @ wr[e * n:(e + 1) * n].t()
            assert _rel(y[b * cap:(b + 1) * cap].cpu(), ref) < 0.012, (fp8, b)


@pytest.mark.parametrize("t,e_local,cap", [(40, 6, 16), (300, 8, 32), (256, 32, 16), (700, 4, 128)])
def test_dynamic_dispatch_and_grouped_gemm(t, e_local, cap):
    torch.manual_seed(t)
    k, dim, n, e0 = 4, 256, 256, 2
    e_total = e_local + 4
    x = torch.randn(t, dim, device=DEV).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(e_total, device=DEV)[:k] for _ in range(t)]).to(torch.int32)
    max_blocks = (t * k + cap - 1) // cap + e_local
    xs = torch.zeros(max_blocks * cap, dim, dtype=torch.bfloat16, device=DEV)
    plan = ops.moe_dispatch_dynamic(x, ids, e0, e_local, cap, xs)
    local = (ids >= e0) & (ids < e0 + e_local)
    assert torch.equal(plan.slot_of >= 0, local)
    counts = torch.stack([(ids == e0 + j).sum() for j in range(e_local)])
    assert int(plan.dyn_blocks) == int(((counts + cap - 1) // cap).sum())
    s = plan.slot_of[local].long()
    assert s.unique().numel() == s.numel()
    blk = torch.div(s, cap, rounding_mode="floor")
    assert torch.equal(plan.block_group[blk].long(), (ids[local] - e0).long())      # a slot's block belongs to its expert
    tok = torch.arange(t, device=DEV)[:, None].expand(t, k)[local]
    assert torch.equal(xs[s], x[tok])
    for fp8 in (False, True):
        w = (torch.randn(e_local * n, dim, device=DEV) * 0.05).to(torch.bfloat16)
        lw = LinearWeight.from_dense(w, fp8=fp8)
        y = ops.grouped_linear_dynamic(xs, lw, e_local, plan)
        N.check_status()
        wr = R.dequant_fp8_weight(lw.weight.cpu(), lw.scale.cpu()) if fp8 else w.float().cpu()
        if fp8:
            xq = ops.quant_fp8_act(xs, tile_rows=cap)
            xr = R.dequant_fp8_act(xq.data.cpu(), xq.scales_fp32().cpu())
        else:
            xr = xs.float().cpu()
        e_of = (ids[local] - e0).long().cpu()
        sc = s.cpu()
        for j in range(0, sc.numel(), max(1, sc.numel() // 50)):     # a sample of the assigned slots
            ref = xr[sc[j]] @ wr[e_of[j] * n:(e_of[j] + 1) * n].t()
            assert _rel(y[sc[j]].cpu(), ref) < 0.015, (fp8, j)


def test_folded_query_projection_matches_q_b_plus_absorb():
    """The second query projection with W_uk folded in (used for up to 256 rows) against q_b followed by
    the per-head absorb, on the same checkpoint tensors, bf16 and fp8."""
    import os
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "benchmarks"))
    import llm_parity
    from hartsyinference_b200 import config
    from hartsyinference_b200.models.llm import config as C
    from hartsyinference_b200.models.llm.mla import fold_q
    from hartsyinference_b200.models.llm.transformer import DecoderModel, ForwardBatch
    # the fold itself against its definition
    heads, nope, rope, k = 3, 128, 64, 96
    qb = torch.randn(heads * (nope + rope), k, device=DEV)
    uk = torch.randn(heads * 512, nope, device=DEV)
    x = torch.randn(5, k, device=DEV)
    f = (x @ fold_q(qb, uk, heads, nope, rope).t()).reshape(5, heads, 576)
    q = (x @ qb.t()).reshape(5, heads, nope + rope)
    want = torch.cat([torch.einsum("thn,hln->thl", q[..., :nope], uk.reshape(heads, 512, nope)), q[..., nope:]], dim=-1)
    assert _rel(f, want) < 1e-4
    mla = C.MlaConfig(q_lora_rank=128, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128)
    cfg = C.tiny("deepseek-v3", vocab_size=512, hidden_size=256, num_heads=16, num_kv_heads=16, head_dim=192, mla=mla,
                 num_layers=2, ffn_size=256, moe=None)
    get = llm_parity._weights(cfg, torch.device(DEV))
    t = 40
    toks = torch.randint(0, cfg.vocab_size, (t,), device=DEV).to(torch.int32)

    def logits(fold, fp8):
        config.set_override("mla_fold_q", fold)
        try:
            m = DecoderModel(cfg, DEV, fp8=fp8)
            m.load_state_dict(get)
        finally:
            config.set_override("mla_fold_q", None)
        assert (m.layers[0].attn_module.w.q_fold is not None) == fold
        m.alloc_kv(4, 16)
        b = ForwardBatch(tokens=toks, positions=torch.arange(t, dtype=torch.int32, device=DEV),
                         slot_mapping=torch.arange(t, dtype=torch.int64, device=DEV),
                         block_table=torch.arange(4, dtype=torch.int32, device=DEV)[None],
                         kv_lens=torch.tensor([t], dtype=torch.int32, device=DEV), is_decode=False,
                         cu_q=torch.tensor([0, t], dtype=torch.int32, device=DEV), max_q_len=t, max_kv_len=t)
        return m.full_logits(m.forward_hidden(b)).float()

    for fp8 in (False, True):
        a, b_ = logits(True, fp8), logits(False, fp8)
        cos = torch.nn.functional.cosine_similarity(a, b_, dim=-1)
        assert float(cos.min()) > (0.99 if fp8 else 0.999), (fp8, cos.min())
