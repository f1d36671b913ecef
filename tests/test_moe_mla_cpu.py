"""Mixture-of-experts and multi-head latent attention on CPU: routing oracle cases, the sharded
modules against dense fp32 oracles, and a toy DeepSeek-style model through the engine."""
from dataclasses import replace

import torch

from hartsyinference_b200 import ops
from hartsyinference_b200.engine import LLMEngine, SamplingParams
from hartsyinference_b200.models.llm import config as C
from hartsyinference_b200.models.llm.mla import MlaAttention, MlaWeights, mla_reference, split_kv_b
from hartsyinference_b200.models.llm.moe import MoeFeedForward, MoeWeights, moe_reference
from hartsyinference_b200.models.llm.transformer import DecoderModel, ForwardBatch
from hartsyinference_b200.ops import LinearWeight
from hartsyinference_b200.ops import reference as R


def _moe_cfg(**kw):
    moe = C.MoeConfig(num_experts=8, top_k=2, expert_ffn=64, num_shared_experts=1, shared_ffn=64,
                      scoring="sigmoid", norm_topk_prob=True, routed_scaling_factor=2.5, n_group=4,
                      topk_group=2, use_correction_bias=True, first_dense_layers=1)
    moe = replace(moe, **kw)
    return C.tiny("deepseek-v3", hidden_size=128, num_heads=4, num_kv_heads=4, moe=moe, num_layers=2)


def test_route_softmax_topk_and_renorm():
    lg = torch.tensor([[0.0, 2.0, 1.0, -1.0], [3.0, 3.0, 0.0, 0.0]])
    ids, w = R.moe_route(lg, None, 2, norm_topk=True)
    assert ids.tolist() == [[1, 2], [0, 1]]                       # tie -> lower index first
    assert torch.allclose(w.sum(-1), torch.ones(2), atol=1e-6)
    ids, w = R.moe_route(lg, None, 2, norm_topk=False)
    assert torch.allclose(w[0], torch.softmax(lg[0], -1)[[1, 2]])


def test_route_group_limited_uses_bias_for_selection_only():
    # 2 groups of 2; the bias lifts group 1 above group 0 although its raw scores are lower
    lg = torch.tensor([[2.0, 1.5, 0.0, -0.5]])
    bias = torch.tensor([0.0, 0.0, 1.0, 1.0])
    ids, w = R.moe_route(lg, bias, 2, n_group=2, topk_group=1, sigmoid=True, norm_topk=False, scale=1.0)
    assert sorted(ids[0].tolist()) == [2, 3]
    assert torch.allclose(w[0], torch.sigmoid(lg[0, ids[0].long()]))   # weights are the unbiased scores


def _full_moe(cfg, seed=0):
    g = torch.Generator().manual_seed(seed)
    m, h = cfg.moe, cfg.hidden_size
    bf = lambda *s: (torch.randn(*s, generator=g) * 0.1).to(torch.bfloat16)
    return {"router": bf(m.num_experts, h), "router_bias": torch.randn(m.num_experts, generator=g) * 0.05,
            "gate_up": bf(m.num_experts, 2 * m.expert_ffn, h), "down": bf(m.num_experts, h, m.expert_ffn),
            "shared_gate_up": bf(2 * m.shared_ffn, h), "shared_down": bf(h, m.shared_ffn)}


def _shard_moe(cfg, full, rank, world):
    m = cfg.moe
    el = m.num_experts // world
    fs = m.shared_ffn // world
    sg, su = full["shared_gate_up"][:m.shared_ffn], full["shared_gate_up"][m.shared_ffn:]
    w = MoeWeights(
        router=LinearWeight(full["router"]), router_bias=full["router_bias"],
        gate_up=LinearWeight(full["gate_up"][rank * el:(rank + 1) * el].reshape(el * 2 * m.expert_ffn, -1).contiguous()),
        down=LinearWeight(full["down"][rank * el:(rank + 1) * el].reshape(el * cfg.hidden_size, -1).contiguous()),
        shared_gate_up=LinearWeight(torch.cat([sg[rank * fs:(rank + 1) * fs], su[rank * fs:(rank + 1) * fs]])),
        shared_down=LinearWeight(full["shared_down"][:, rank * fs:(rank + 1) * fs].contiguous()))
    return MoeFeedForward(cfg, w, rank, world)


def test_moe_module_matches_dense_oracle_and_expert_parallel_sum():
    cfg = _moe_cfg()
    full = _full_moe(cfg)
    h = (torch.randn(11, cfg.hidden_size) * 0.5).to(torch.bfloat16)
    ref = moe_reference(h, cfg, full)
    one = _shard_moe(cfg, full, 0, 1)(h).float()
    assert (one - ref).abs().max() < 0.03 * ref.abs().max() + 1e-3
    # two ranks: each computes its experts + its slice of the shared expert; the sum is the output
    parts = [_shard_moe(cfg, full, r, 2)(h).float() for r in range(2)]
    assert (parts[0] + parts[1] - ref).abs().max() < 0.04 * ref.abs().max() + 1e-3


def test_moe_long_input_is_chunked():
    cfg = _moe_cfg(n_group=1, topk_group=1, use_correction_bias=False)
    full = _full_moe(cfg, 3)
    full["router_bias"] = None
    h = (torch.randn(150, cfg.hidden_size) * 0.5).to(torch.bfloat16)
    out = _shard_moe(cfg, full, 0, 1)(h).float()
    ref = moe_reference(h, cfg, full)
    assert (out - ref).abs().max() < 0.03 * ref.abs().max() + 1e-3


def _mla_setup(q_lora=True, seed=0):
    mla = C.MlaConfig(q_lora_rank=96 if q_lora else 0, kv_lora_rank=512, qk_nope_head_dim=32, qk_rope_head_dim=64,
                      v_head_dim=32)
    cfg = C.tiny("deepseek-v3", hidden_size=128, num_heads=4, num_kv_heads=4, head_dim=96, mla=mla, moe=None,
                 num_layers=1)
    g = torch.Generator().manual_seed(seed)
    bf = lambda *s: (torch.randn(*s, generator=g) * 0.08).to(torch.bfloat16)
    heads, dq = cfg.num_heads, 96
    full = {"kv_a": bf(576, 128), "kv_a_norm": torch.ones(512, dtype=torch.bfloat16),
            "kv_b": bf(heads * (32 + 32), 512), "o": bf(128, heads * 32)}
    if q_lora:
        full.update({"q_a": bf(96, 128), "q_a_norm": torch.ones(96, dtype=torch.bfloat16), "q_b": bf(heads * dq, 96)})
    else:
        full["q"] = bf(heads * dq, 128)
    return cfg, full


def _mla_module(cfg, full, rank=0, world=1):
    m = cfg.mla
    hl = cfg.num_heads // world
    dq, per = 96, 64
    kv_b = full["kv_b"][rank * hl * per:(rank + 1) * hl * per]
    w_uk, w_uv = split_kv_b(kv_b, hl, 32, 32)
    qb = full["q_b"] if "q_b" in full else full["q"]
    w = MlaWeights(q_a=LinearWeight(full["q_a"]) if "q_a" in full else None, q_a_norm=full.get("q_a_norm"),
                   q_b=LinearWeight(qb[rank * hl * dq:(rank + 1) * hl * dq].contiguous()),
                   kv_a=LinearWeight(full["kv_a"]), kv_a_norm=full["kv_a_norm"],
                   w_uk=LinearWeight(w_uk.contiguous()), w_uv=LinearWeight(w_uv.contiguous()),
                   o=LinearWeight(full["o"][:, rank * hl * 32:(rank + 1) * hl * 32].contiguous()))
    return MlaAttention(cfg, w, hl)


class _FakeModel:
    def __init__(self, cfg, pages=8, page=16):
        self.cfg = cfg
        self.kv_cache = torch.zeros(1, pages, page, 576, dtype=torch.bfloat16)
        self.inv_freq = R.rope_inv_freq(64, cfg.rope_theta)
        self.rope_attn_factor = 1.0

    def _reduce_linear(self, x, w):
        return ops.linear(x, w)


def _prefill_batch(t, page=16):
    pos = torch.arange(t, dtype=torch.int32)
    npg = (t + page - 1) // page
    table = torch.arange(1, npg + 1, dtype=torch.int32).unsqueeze(0)      # pages 1..npg
    slots = (table[0, (pos // page).long()].long() * page + (pos % page).long())
    return ForwardBatch(tokens=None, positions=pos, slot_mapping=slots, block_table=table,
                        kv_lens=torch.tensor([t], dtype=torch.int32), cu_q=torch.tensor([0, t], dtype=torch.int32),
                        max_q_len=t, is_decode=False, max_kv_len=t)


def test_mla_absorbed_prefill_matches_expanded_oracle():
    for q_lora in (True, False):
        cfg, full = _mla_setup(q_lora)
        mod = _mla_module(cfg, full)
        model = _FakeModel(cfg)
        t = 21
        h = (torch.randn(t, 128) * 0.5).to(torch.bfloat16)
        batch = _prefill_batch(t)
        out = mod(h, batch, 0, model).float()
        ref = mla_reference(h, batch.positions, cfg, full, model.inv_freq, mod.scale(model))
        assert (out - ref).abs().max() < 0.03 * ref.abs().max() + 2e-3


def test_mla_decode_after_prefill_and_head_sharding():
    cfg, full = _mla_setup(True, seed=2)
    t = 19
    h = (torch.randn(t + 1, 128) * 0.5).to(torch.bfloat16)
    ref = mla_reference(h, torch.arange(t + 1, dtype=torch.int32), cfg, full, R.rope_inv_freq(64, cfg.rope_theta),
                        1.0 / 96 ** 0.5)
    total = torch.zeros(128)
    for rank in range(2):
        mod = _mla_module(cfg, full, rank, 2)
        model = _FakeModel(cfg)
        batch = _prefill_batch(t)
        mod(h[:t], batch, 0, model)
        # one decode step for the next token, reading the latent cache written by the prefill
        page = 16
        pos = torch.tensor([t], dtype=torch.int32)
        table = torch.arange(1, (t + 1 + page - 1) // page + 1, dtype=torch.int32).unsqueeze(0)
        slot = (table[0, t // page].long() * page + t % page).reshape(1)
        dec = ForwardBatch(tokens=None, positions=pos, slot_mapping=slot, block_table=table,
                           kv_lens=torch.tensor([t + 1], dtype=torch.int32), cu_q=None, max_q_len=1,
                           is_decode=True, max_kv_len=t + 1)
        total += mod(h[t:], dec, 0, model).float()[0]
    assert (total - ref[-1]).abs().max() < 0.04 * ref.abs().max() + 2e-3


def test_toy_deepseek_generates_through_the_engine():
    mla = C.MlaConfig(q_lora_rank=64, kv_lora_rank=512, qk_nope_head_dim=32, qk_rope_head_dim=64, v_head_dim=32)
    cfg = replace(_moe_cfg(), mla=mla, head_dim=96)
    model = DecoderModel(cfg, "cpu")
    model.random_init(0, std=0.05)
    assert model.layers[0].ffn_module is None and model.layers[1].ffn_module is not None
    assert model.layers[0].attn_module is not None
    eng = LLMEngine(model, num_pages=32, page_size=16, max_batch=4, prefill_chunk=64, max_model_len=128)
    a = eng.generate([[5, 6, 7, 8, 9]], SamplingParams(greedy=True, max_tokens=6))[0]
    # the same prompt decoded again after the cache was reused gives the same tokens
    b = eng.generate([[5, 6, 7, 8, 9]], SamplingParams(greedy=True, max_tokens=6))[0]
    assert len(a) == 6 and a == b
    assert model.kv_bytes_per_page(16) == cfg.num_layers * 16 * 576 * 2
