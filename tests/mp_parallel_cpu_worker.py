"""CPU ranks over gloo: tensor-parallel decoder, tensor-parallel Flux, Ulysses Wan and CFG-parallel
pipelines must reproduce the single-rank result (tolerance = bf16 rounding of different summation
orders). Launched by tests/test_parallel_cpu.py under torchrun."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

from hartsyinference_b200.models.dit import flux as F
from hartsyinference_b200.models.dit import wan as W
from hartsyinference_b200.models.llm import config as C
from hartsyinference_b200.models.llm.transformer import DecoderModel, ForwardBatch
from hartsyinference_b200.parallel import init_comm


def cos(a, b):
    return torch.nn.functional.cosine_similarity(a.float().flatten(), b.float().flatten(), dim=0).item()


def main():
    comm = init_comm("gloo")
    rank, world = comm.rank, comm.world
    # ---- TP decoder vs single
    cfg = C.tiny("llama-3-70b", vocab_size=256, hidden_size=128, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=32, ffn_size=256)
    g = torch.Generator().manual_seed(3)
    full = {}
    mk = lambda n, *s: full.__setitem__(n, (torch.randn(*s, generator=g) * 0.05).to(torch.bfloat16))
    mk("model.embed_tokens.weight", 256, 128); mk("lm_head.weight", 256, 128)
    full["model.norm.weight"] = torch.ones(128, dtype=torch.bfloat16)
    for i in range(2):
        p = f"model.layers.{i}."
        mk(p + "self_attn.q_proj.weight", 128, 128); mk(p + "self_attn.k_proj.weight", 64, 128); mk(p + "self_attn.v_proj.weight", 64, 128)
        mk(p + "self_attn.o_proj.weight", 128, 128); mk(p + "mlp.gate_proj.weight", 256, 128); mk(p + "mlp.up_proj.weight", 256, 128)
        mk(p + "mlp.down_proj.weight", 128, 256)
        full[p + "input_layernorm.weight"] = torch.ones(128, dtype=torch.bfloat16)
        full[p + "post_attention_layernorm.weight"] = torch.ones(128, dtype=torch.bfloat16)
    t = 20
    toks = torch.randint(0, 256, (t,), generator=g).to(torch.int32)

    def run(m):
        m.alloc_kv(4, 16)
        b = ForwardBatch(tokens=toks, positions=torch.arange(t, dtype=torch.int32), slot_mapping=torch.arange(t, dtype=torch.int64),
                         block_table=torch.arange(4, dtype=torch.int32)[None], kv_lens=torch.tensor([t], dtype=torch.int32),
                         is_decode=False, cu_q=torch.tensor([0, t], dtype=torch.int32), max_q_len=t, max_kv_len=t)
        hid = m.forward_hidden(b)
        return m.full_logits(hid), m.greedy_tokens(hid[-1:])

    single = DecoderModel(cfg, "cpu"); single.load_state_dict(full.get)
    tp = DecoderModel(cfg, "cpu", comm=comm); tp.load_state_dict(full.get)
    (ls, ts), (lt, tt) = run(single), run(tp)
    assert cos(ls, lt) > 0.999, cos(ls, lt)
    assert int(ts) == int(tt) or abs(float(ls[-1, int(ts)]) - float(ls[-1, int(tt)])) < 0.05
    # ---- layer-split pipeline vs single: stage 0 holds layer 0, stage 1 layer 1 + head; generation
    # through one engine per stage gives the single-process tokens
    from hartsyinference_b200.engine import LLMEngine, SamplingParams
    from hartsyinference_b200.parallel.pipeline import PipelinedModel, split_layers
    assert split_layers(7, 3, [1, 1, 2]) == [(0, 2), (2, 4), (4, 7)]
    pp = PipelinedModel(cfg, comm, "cpu")
    pp.load_state_dict(full.get)
    assert len(pp.model.layers) == 1
    lp, tpk = run(pp)
    assert cos(ls, lp) > 0.9999, cos(ls, lp)
    assert int(tpk) == int(ts)
    prompts = [toks.tolist(), toks[:7].tolist()]
    sp = SamplingParams(greedy=True, max_tokens=6, ignore_eos=True)
    ref_out = LLMEngine(single, num_pages=16, page_size=16, max_batch=4, prefill_chunk=64, max_model_len=64).generate(prompts, sp)
    pp_out = LLMEngine(pp, num_pages=16, page_size=16, max_batch=4, prefill_chunk=64, max_model_len=64).generate(prompts, sp)
    assert pp_out == ref_out, (pp_out, ref_out)
    # micro-batches: a batch of four sequences is cut in two, stage 1 works on the first half while
    # stage 0 computes the second; prefill (cut at a sequence boundary) and decode steps both split
    pp2 = PipelinedModel(cfg, comm, "cpu", micro_batches=2)
    pp2.load_state_dict(full.get)
    prompts4 = [toks.tolist(), toks[:7].tolist(), toks[3:12].tolist(), toks[:5].tolist()]
    ref4 = LLMEngine(single, num_pages=32, page_size=16, max_batch=4, prefill_chunk=64, max_model_len=64).generate(prompts4, sp)
    eng2 = LLMEngine(pp2, num_pages=32, page_size=16, max_batch=4, prefill_chunk=64, max_model_len=64)
    seen = []
    orig_split = pp2.split_batch
    pp2.split_batch = lambda b: (lambda parts: (seen.append((b.is_decode, len(parts))), parts)[1])(orig_split(b))
    out4 = eng2.generate(prompts4, sp)
    assert out4 == ref4, (out4, ref4)
    assert (True, 2) in seen and (False, 2) in seen, seen
    # ---- TP Flux vs single (same seed => same full weights, sharded per rank)
    fcfg = F.tiny_flux(num_heads=4, head_dim=32)
    gi = torch.Generator().manual_seed(5)
    img = torch.randn(1, 16, fcfg.in_channels, generator=gi); txt = torch.randn(1, 6, fcfg.context_dim, generator=gi)
    pooled = torch.randn(1, fcfg.pooled_dim, generator=gi)
    ii, it = F.flux_ids(4, 4, 6)
    args = (img, txt, torch.tensor([0.6]), pooled, ii, it, torch.tensor([3.5]))
    f1 = F.FluxTransformer(fcfg, "cpu", seed=9).forward(*args)
    f2 = F.FluxTransformer(fcfg, "cpu", comm=comm, seed=9).forward(*args)
    assert cos(f1, f2) > 0.999, cos(f1, f2)
    # ---- Ulysses Wan vs single
    wcfg = W.tiny_wan()
    lat = torch.randn(16, 2, 4, 4, generator=gi)
    ctxr = torch.randn(wcfg.text_len, wcfg.text_dim, generator=gi)
    w1 = W.WanTransformer(wcfg, "cpu", seed=11)
    w2 = W.WanTransformer(wcfg, "cpu", sp_comm=comm, seed=11)
    o1 = w1.forward(lat, torch.tensor(300.0), w1.encode_text(ctxr))
    o2 = w2.forward(lat, torch.tensor(300.0), w2.encode_text(ctxr))
    assert cos(o1, o2) > 0.999, cos(o1, o2)
    # ---- head count that does not divide by the group: keys / values are gathered instead (context parallel)
    if world == 2:
        odd = W.tiny_wan(hidden_size=96, num_heads=3, head_dim=32)
        a1 = W.WanTransformer(odd, "cpu", seed=13)
        a2 = W.WanTransformer(odd, "cpu", sp_comm=comm, seed=13)
        assert not a2.ulysses
        ctxo = torch.randn(odd.text_len, odd.text_dim, generator=gi)
        r1 = a1.forward(lat, torch.tensor(300.0), a1.encode_text(ctxo))
        r2 = a2.forward(lat, torch.tensor(300.0), a2.encode_text(ctxo))
        assert cos(r1, r2) > 0.999, cos(r1, r2)
    # ---- CFG-parallel pipelines vs sequential CFG
    from hartsyinference_b200.pipelines.flux import FluxComponents, FluxPipeline
    from hartsyinference_b200.pipelines.wan import WanComponents, WanPipeline
    fx = F.FluxTransformer(fcfg, "cpu", seed=9)
    c, pl = torch.randn(6, fcfg.context_dim, generator=gi), torch.randn(fcfg.pooled_dim, generator=gi)
    n = (torch.randn(6, fcfg.context_dim, generator=gi), torch.randn(fcfg.pooled_dim, generator=gi))
    zs = FluxPipeline(FluxComponents(fx)).denoise(c, pl, 64, 64, 3, 3.5, 1, n, 2.0)
    zp = FluxPipeline(FluxComponents(fx), cfg_comm=comm).denoise(c, pl, 64, 64, 3, 3.5, 1, n, 2.0)
    assert cos(zs, zp) > 0.9999, cos(zs, zp)
    ws = WanPipeline(WanComponents(w1)).denoise(ctxr, ctxr * 0.5, 5, 32, 32, 3, 3.0, 7)
    wp = WanPipeline(WanComponents(w1), cfg_comm=comm).denoise(ctxr, ctxr * 0.5, 5, 32, 32, 3, 3.0, 7)
    assert cos(ws, wp) > 0.9999, cos(ws, wp)
    comm.barrier()
    if rank == 0:
        print("PARALLEL_CPU_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
