"""Ranks over gloo (CPU) or NCCL (one GPU each): a toy DeepSeek-style model (latent attention, routed
+ shared experts, one leading dense layer) in the data-parallel-attention layout must reproduce the
single-rank model: prefill in the tensor-parallel layout, then decode steps with the requests dealt
over the ranks, both by logits and through the engine. Launched under torchrun by
tests/test_dp_attention.py (CPU) and tests/test_fused_tp_gpu.py (GPUs)."""
import os
import sys
from dataclasses import replace

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "benchmarks"))

import torch

from hartsyinference_b200.engine import LLMEngine, SamplingParams
from hartsyinference_b200.models.llm import config as C
from hartsyinference_b200.models.llm.transformer import DecoderModel, ForwardBatch
from hartsyinference_b200.parallel import init_comm
from hartsyinference_b200.parallel.dp_attention import enable_dp_attention


def main():
    gpu = torch.cuda.is_available() and os.environ.get("DP_WORKER_DEVICE", "cuda") == "cuda"
    comm = init_comm("nccl" if gpu else "gloo")
    rank, world = comm.rank, comm.world
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0))) if gpu else torch.device("cpu")
    if gpu:
        torch.cuda.set_device(dev)
    import llm_parity
    from hartsyinference_b200.ops import _native as N
    moe = C.MoeConfig(num_experts=8, top_k=2, expert_ffn=128, num_shared_experts=1, shared_ffn=128,
                      scoring="sigmoid", norm_topk_prob=True, routed_scaling_factor=2.5, n_group=4,
                      topk_group=2, use_correction_bias=True, first_dense_layers=1)
    cfg = C.tiny("deepseek-v3", vocab_size=512, hidden_size=256, num_heads=4 * world, num_kv_heads=4 * world, moe=moe,
                 num_layers=3, ffn_size=256)
    get = llm_parity._weights(cfg, dev)
    seqs, plen, page = 2 * world, 9, 16
    g = torch.Generator().manual_seed(5)
    prompts = torch.randint(0, cfg.vocab_size, (seqs, plen), generator=g).to(torch.int32)

    def run(model):
        """Prefill all sequences (one page each), then two decode steps; returns the decode logits."""
        model.alloc_kv(seqs + 1, page)
        tok = prompts.reshape(-1).to(dev)
        pos = torch.arange(plen, dtype=torch.int32).repeat(seqs).to(dev)
        slots = (torch.arange(seqs)[:, None] * page + torch.arange(plen)[None]).reshape(-1).to(torch.int64).to(dev)
        table = torch.arange(seqs, dtype=torch.int32)[:, None].to(dev)
        b = ForwardBatch(tokens=tok, positions=pos, slot_mapping=slots, block_table=table,
                         kv_lens=torch.full((seqs,), plen, dtype=torch.int32, device=dev), is_decode=False,
                         cu_q=(torch.arange(seqs + 1, dtype=torch.int32) * plen).to(dev), max_q_len=plen, max_kv_len=plen)
        hid = model.forward_hidden(b)
        nxt = model.full_logits(hid[plen - 1::plen]).float().argmax(-1).to(torch.int32)
        outs = []
        for step in range(2):
            n = plen + step
            b = ForwardBatch(tokens=nxt, positions=torch.full((seqs,), n, dtype=torch.int32, device=dev),
                             slot_mapping=(torch.arange(seqs) * page + n).to(torch.int64).to(dev), block_table=table,
                             kv_lens=torch.full((seqs,), n + 1, dtype=torch.int32, device=dev), is_decode=True,
                             max_q_len=1, max_kv_len=n + 1)
            lg = model.full_logits(model.forward_hidden(b)).float()
            outs.append(lg)
            nxt = first_tokens[step] if first_tokens else lg.argmax(-1).to(torch.int32)
            if not first_tokens:
                chosen.append(nxt)
        return outs

    first_tokens, chosen = [], []
    for fused in ([False, True] if gpu else [False]):
        sharded = DecoderModel(cfg, dev, comm=comm, dp_attention=True)
        sharded.load_state_dict(get)
        assert all(lw.attn_dp is not None for lw in sharded.layers)
        assert enable_dp_attention(sharded, comm, max_rows=seqs, fused=fused) == fused
        calls = []
        orig = sharded._forward_dp_attention
        sharded._forward_dp_attention = lambda b: (calls.append(b.tokens.shape[0]), orig(b))[1]
        chosen.clear()
        got = run(sharded)
        assert calls == [seqs, seqs], calls            # both decode steps, not the prefill
        if gpu:
            N.check_status(dev)
        # every rank's cache holds every request's rows, including the ones other ranks wrote at decode
        mine = sharded.kv_cache[1].view(-1, 576)[torch.arange(seqs, device=dev) * page + plen].float()
        assert bool((mine.abs().sum(-1) > 0).all())
        first_tokens = list(chosen)
        single = DecoderModel(cfg, dev)
        single.load_state_dict(get)
        want = run(single)
        for a, b_ in zip(got, want):
            cos = torch.nn.functional.cosine_similarity(a, b_, dim=-1)
            assert float(cos.min()) > 0.995, (fused, cos)
        ref_cache = single.kv_cache[1].view(-1, 576)[torch.arange(seqs, device=dev) * page + plen].float()
        assert float(torch.nn.functional.cosine_similarity(mine, ref_cache, dim=-1).min()) > 0.99
        # through the engine (scheduler, paged cache, CUDA graphs on GPUs): same greedy tokens as one rank
        sp = SamplingParams(greedy=True, max_tokens=5, ignore_eos=True)
        pl = [p.tolist() for p in prompts]
        kw = dict(num_pages=4 * seqs, page_size=16, max_batch=seqs, prefill_chunk=64, max_model_len=48)
        out_dp = LLMEngine(sharded, **kw).generate(pl, sp)
        out_one = LLMEngine(single, **kw).generate(pl, sp)
        agree = sum(x == y for a, b_ in zip(out_dp, out_one) for x, y in zip(a, b_)) / (5 * seqs)
        assert agree >= 0.8, (fused, agree, out_dp, out_one)
        first_tokens = []
        if gpu:
            N.check_status(dev)
        comm.barrier()
        sharded.dp_exchange.close()
        del sharded, single
    if rank == 0:
        print("DP_ATTENTION_OK", flush=True)


if __name__ == "__main__":
    main()
