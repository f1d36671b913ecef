"""Worker of the multi-GPU fused tensor-parallel test (one process per GPU under torchrun).

Checks (1) the fused GEMM + all-reduce + residual + RMSNorm + fp8-emit kernel against a NCCL
all-reduce of the plain GEMM followed by the same math in fp32, (2) the stand-alone all-reduce and
CFG-combine kernels, and (3) that a tensor-parallel toy decoder produces the same logits as the
single-GPU model built from the same full weights, through both the NCCL path and the fused path."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

from hartsyinference_b200 import ops
from hartsyinference_b200.models.llm import config as C
from hartsyinference_b200.models.llm.transformer import DecoderModel, ForwardBatch
from hartsyinference_b200.ops import _native as N
from hartsyinference_b200.ops import reference as R
from hartsyinference_b200.parallel import init_comm
from hartsyinference_b200.parallel.fused import FusedColumnParallel, FusedRowParallel, enable_fused_tp


def rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-6)).item()


def main():
    comm = init_comm()
    rank, world = comm.rank, comm.world
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.manual_seed(100 + rank)
    fused = FusedRowParallel(comm, 2048, dev)
    if rank == 0:
        print("heap transport", fused.heap.transport, "multicast", fused.use_mc, flush=True)
    for fp8 in (False, True):
        for m in (64, 5, 128, 1):
            n, k = 2048, 1024
            x = (torch.randn(m, k, device=dev) * 0.5).to(torch.bfloat16)
            w = ops.LinearWeight.from_dense((torch.randn(n, k, device=dev) * 0.2).to(torch.bfloat16), fp8=fp8)
            res0 = torch.randn(m, n, device=dev).to(torch.bfloat16)
            nw = (1 + 0.1 * torch.randn(n, device=dev)).to(torch.bfloat16)
            dist.broadcast(res0, 0)
            dist.broadcast(nw, 0)
            res = res0.clone()
            h, h8 = fused(x, w, res=res, norm_w=nw, eps=1e-5, emit_bf16=True, emit_fp8=True)
            h = h.clone()
            deq = R.dequant_fp8_act(h8.data.clone(), h8.scales_fp32())
            part = ops.linear(x, w, splits=1).float()
            dist.all_reduce(part)
            rr = (part.to(torch.bfloat16).float() + res0.float()).to(torch.bfloat16).float()
            want = rr * torch.rsqrt((rr * rr).mean(-1, keepdim=True) + 1e-5) * nw.float()
            N.check_status(dev)
            per = (m + world - 1) // world
            own = slice(min(m, rank * per), min(m, (rank + 1) * per))
            assert rel(h, want) < 1.5e-2, (fp8, m, "norm", rel(h, want))
            assert rel(deq, want) < 6e-2, (fp8, m, "fp8", rel(deq, want))
            if own.stop > own.start:
                assert rel(res[own], rr[own]) < 1.5e-2, (fp8, m, "residual", rel(res[own], rr[own]))
            # rows of other ranks are left alone
            other = torch.ones(m, dtype=torch.bool, device=dev)
            other[own] = False
            assert torch.equal(res[other], res0[other])
            y, _ = fused(x, w)                                   # plain all-reduced linear
            assert rel(y, part) < 1.5e-2, (fp8, m, "plain", rel(y, part))
    # ---- more than 128 tokens: GEMM + all-reduce + gated residual in one kernel
    big = FusedRowParallel(comm, 1024, dev, max_large_tokens=1200)
    for fp8 in (False, True):
        for m in (1100, 300):
            n, k = 1024, 512
            x = (torch.randn(m, k, device=dev) * 0.5).to(torch.bfloat16)
            w = ops.LinearWeight.from_dense((torch.randn(n, k, device=dev) * 0.2).to(torch.bfloat16),
                                            torch.randn(n, device=dev).to(torch.bfloat16), fp8=fp8)
            res = torch.randn(m, n, device=dev).to(torch.bfloat16)
            gate = torch.randn(n, device=dev).to(torch.bfloat16)
            dist.broadcast(res, 0)
            dist.broadcast(gate, 0)
            part = ops.linear(x, w).float()                      # includes this rank's bias
            dist.all_reduce(part)
            # every rank added its own bias in `part`; the fused kernel adds the bias once (rank-local bias tensor of the owner)
            want = None
            for it in range(3):
                y = big.large(x, w, res=res, gate=gate, slot=it % 2).clone()
                N.check_status(dev)
                bias_all = w.bias.float().clone()
                dist.all_reduce(bias_all)
                # owner-row bias: rows owned by rank r carry rank r's bias
                per = (m + world - 1) // world
                wb = torch.zeros(m, n, device=dev)
                biases = [torch.zeros_like(w.bias) for _ in range(world)]
                dist.all_gather(biases, w.bias)
                for r in range(world):
                    wb[r * per:(r + 1) * per] = biases[r].float()
                want = res.float() + gate.float() * (part - bias_all + wb)
                assert rel(y, want) < 1.5e-2, ("large", fp8, m, it, rel(y, want))
    # ---- a sequence-parallel MLP: all-gather -> GEMM (column-parallel, gelu), GEMM -> reduce-scatter
    # (row-parallel, gated residual on the rank's rows), against the same MLP on one GPU
    colp = FusedColumnParallel(comm, 1200, 1024, dev)
    gen = torch.Generator(device="cpu").manual_seed(21)
    for fp8 in (False, True):
        for m in (1100, 300):
            hdim, fdim = 1024, 2048
            x_full = (torch.randn(m, hdim, generator=gen) * 0.5).to(torch.bfloat16).to(dev)       # same on all ranks
            w1 = (torch.randn(fdim, hdim, generator=gen) * 0.05).to(torch.bfloat16).to(dev)
            w2 = (torch.randn(hdim, fdim, generator=gen) * 0.05).to(torch.bfloat16).to(dev)
            b1 = torch.randn(fdim, generator=gen).to(torch.bfloat16).to(dev)
            gate = torch.randn(hdim, generator=gen).to(torch.bfloat16).to(dev)
            fl = fdim // world
            lw1 = ops.LinearWeight.from_dense(w1[rank * fl:(rank + 1) * fl].contiguous(), b1[rank * fl:(rank + 1) * fl].contiguous(), fp8=fp8)
            lw2 = ops.LinearWeight.from_dense(w2[:, rank * fl:(rank + 1) * fl].contiguous(), fp8=fp8)
            a, b = colp.owned_rows(m)
            for it in range(2):
                h = colp(x_full[a:b].contiguous(), lw1, m, act="gelu_tanh")                         # [m, fl]
                out = torch.empty(b - a, hdim, dtype=torch.bfloat16, device=dev)
                big.large(h, lw2, res=x_full[a:b].contiguous(), gate=gate, scatter_out=out)
                N.check_status(dev)
                hh = torch.nn.functional.gelu(x_full.float() @ w1.float().t() + b1.float(), approximate="tanh").to(torch.bfloat16).float()
                want = x_full.float() + gate.float() * (hh @ w2.float().t())
                assert rel(out, want[a:b]) < (6e-2 if fp8 else 2e-2), ("sp-mlp", fp8, m, it, rel(out, want[a:b]))
    comm.barrier()
    colp.close()
    comm.barrier()
    big.close()
    # ---- peer-memory all-reduce kernel vs NCCL, eager and under a CUDA graph
    from hartsyinference_b200.parallel.custom_ar import CustomAllReduce
    car = CustomAllReduce(comm, 128 * 2048, dev)
    for m, n in ((64, 2048), (1, 256), (128, 2048), (7, 512)):
        for it in range(3):
            x = torch.randn(m, n, device=dev).to(torch.bfloat16)
            want = x.float().clone()
            dist.all_reduce(want)
            car.input(m, n).copy_(x)
            got = car.reduce(m, n).float()
            N.check_status(dev)
            assert rel(got, want) < 8e-3, (m, n, it, rel(got, want))
            res = torch.randn(m, n, device=dev).to(torch.bfloat16)
            dist.broadcast(res, 0)             # the residual stream is replicated over the group
            car.input(m, n).copy_(x)
            got = car.reduce(m, n, residual=res).float()
            assert rel(got, want + res.float()) < 8e-3
    x = torch.randn(64, 2048, device=dev).to(torch.bfloat16)
    car.input(64, 2048).copy_(x)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        y1 = car.reduce(64, 2048)
        car.input(64, 2048).copy_(y1)
        y2 = car.reduce(64, 2048)
    want = x.float().clone()
    dist.all_reduce(want)
    want = want.to(torch.bfloat16).float() * world
    for _ in range(3):
        car.input(64, 2048).copy_(x)
        g.replay()
        torch.cuda.synchronize()
        assert rel(y2.float(), want) < 1e-2
    N.check_status(dev)
    car.close()
    # ---- CFG-parallel combine fused with the Euler step (ranks 0 / 1 = conditional / unconditional)
    if world == 2:
        from hartsyinference_b200.parallel.cfg_combine import FusedCfgCombine
        fc = FusedCfgCombine(comm, 4096 * 64, dev)
        gen = torch.Generator(device="cpu").manual_seed(5)
        z0 = torch.randn(4096 * 64, generator=gen)
        for it in range(4):
            preds = [(torch.randn(4096 * 64, generator=gen) * 0.5).to(torch.bfloat16) for _ in range(2)]   # same on both ranks
            z = z0.clone().to(dev)
            fc.step(z, preds[rank].to(dev), 3.5, -0.05)
            want = z0 + (3.5 * preds[0].float() + (1 - 3.5) * preds[1].float()) * -0.05
            N.check_status(dev)
            assert (z.cpu() - want).abs().max() < 1e-5, (it, (z.cpu() - want).abs().max())
            z0 = want
        # the guided prediction by itself (fp32 slots), for schedulers that are not an Euler step
        pf = [torch.randn(4096 * 64, generator=gen) for _ in range(2)]
        v = fc.combine(pf[rank].to(dev), 5.0)
        N.check_status(dev)
        assert (v.cpu() - (5.0 * pf[0] + (1 - 5.0) * pf[1])).abs().max() < 1e-5
        fc.close()
    # ---- sequence-parallel attention with the exchange fused into the kernels, vs fp32 over the full sequence
    from hartsyinference_b200.parallel.ulysses import FusedUlyssesAttention
    # head counts: one the group divides (head split), and one it does not (K / V to every rank)
    for heads, int8, s_l in [(2 * world, False, 192), (2 * world, False, 100), (2 * world, True, 192), (2 * world, True, 100),
                             (world + 1, False, 192), (world + 1, True, 100)]:
        if True:
            gen = torch.Generator(device="cpu").manual_seed(11 + s_l)
            q, k, v = (torch.randn(world * s_l, heads, 128, generator=gen).to(torch.bfloat16).to(dev) for _ in range(3))   # same on all ranks
            sc = torch.einsum("qhd,khd->hqk", q.float(), k.float()) * 128 ** -0.5
            want = torch.einsum("hqk,khd->qhd", torch.softmax(sc, -1), v.float()).reshape(world * s_l, -1)
            fu = FusedUlyssesAttention(comm, s_l, heads, dev, int8=int8)
            assert fu.context_parallel == (heads % world != 0)
            if not int8 and heads % world != 0:
                # the same case with K / V read from their owners by the attention kernel (over NVLink here)
                fp = FusedUlyssesAttention(comm, s_l, heads, dev, pull=True)
                mine_p = slice(rank * s_l, (rank + 1) * s_l)
                for it in range(2):
                    got_p = fp(q[mine_p].contiguous(), k[mine_p].contiguous(), v[mine_p].contiguous()).clone()
                    N.check_status(dev)
                    assert rel(got_p, want[mine_p]) < 0.02, ("pull", heads, s_l, it, rel(got_p, want[mine_p]))
                comm.barrier()
                fp.close()
            mine = slice(rank * s_l, (rank + 1) * s_l)
            for it in range(3):
                got = fu(q[mine].contiguous(), k[mine].contiguous(), v[mine].contiguous()).clone()
                N.check_status(dev)
                assert rel(got, want[mine]) < (0.06 if int8 else 0.02), ("ulysses", heads, int8, s_l, it, rel(got, want[mine]))
            comm.barrier()
            fu.close()
    if rank == 0:
        print("ULYSSES_OK", flush=True)
    # ---- TP model vs single-GPU model
    cfg = C.tiny("llama-3-70b", vocab_size=1024, hidden_size=512, num_layers=2, num_heads=8, num_kv_heads=2,
                 head_dim=128, ffn_size=1024)
    g = torch.Generator().manual_seed(7)
    full = {}

    def mk(name, *shape, std=0.05):
        full[name] = (torch.randn(*shape, generator=g) * std).to(torch.bfloat16)

    mk("model.embed_tokens.weight", cfg.vocab_size, cfg.hidden_size)
    mk("lm_head.weight", cfg.vocab_size, cfg.hidden_size)
    full["model.norm.weight"] = torch.ones(cfg.hidden_size, dtype=torch.bfloat16)
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}."
        mk(p + "self_attn.q_proj.weight", cfg.q_size, cfg.hidden_size)
        mk(p + "self_attn.k_proj.weight", cfg.kv_size, cfg.hidden_size)
        mk(p + "self_attn.v_proj.weight", cfg.kv_size, cfg.hidden_size)
        mk(p + "self_attn.o_proj.weight", cfg.hidden_size, cfg.q_size)
        mk(p + "mlp.gate_proj.weight", cfg.ffn_size, cfg.hidden_size)
        mk(p + "mlp.up_proj.weight", cfg.ffn_size, cfg.hidden_size)
        mk(p + "mlp.down_proj.weight", cfg.hidden_size, cfg.ffn_size)
        full[p + "input_layernorm.weight"] = torch.ones(cfg.hidden_size, dtype=torch.bfloat16)
        full[p + "post_attention_layernorm.weight"] = torch.ones(cfg.hidden_size, dtype=torch.bfloat16)
    t = 48
    toks = torch.randint(0, cfg.vocab_size, (t,), generator=g).to(torch.int32)

    def run(model):
        model.alloc_kv(8, 16)
        b = ForwardBatch(tokens=toks.to(dev), positions=torch.arange(t, dtype=torch.int32, device=dev),
                         slot_mapping=torch.arange(t, dtype=torch.int64, device=dev),
                         block_table=torch.arange(8, dtype=torch.int32, device=dev)[None],
                         kv_lens=torch.tensor([t], dtype=torch.int32, device=dev), is_decode=False,
                         cu_q=torch.tensor([0, t], dtype=torch.int32, device=dev), max_q_len=t, max_kv_len=t)
        return model.full_logits(model.forward_hidden(b)).float()

    single = DecoderModel(cfg, dev)
    single.load_state_dict(full.get)
    ref = run(single)
    tp = DecoderModel(cfg, dev, comm=comm)
    tp.load_state_dict(full.get)
    got = run(tp)
    cos = torch.nn.functional.cosine_similarity(got, ref, dim=-1).min().item()
    assert cos > 0.999, ("nccl", cos)
    assert enable_fused_tp(tp, comm)
    assert tp._fused_tp_ok(t)
    got2 = run(tp)
    N.check_status(dev)
    cos2 = torch.nn.functional.cosine_similarity(got2, ref, dim=-1).min().item()
    assert cos2 > 0.999, ("fused", cos2)
    tok_a = tp.greedy_tokens(tp.forward_hidden.__self__.final_norm[None].expand(1, -1).contiguous() * 0 + 1)
    comm.barrier()
    torch.cuda.synchronize()
    fused.close()
    tp.fused_rp.close()
    comm.barrier()
    if rank == 0:
        print("FUSED_TP_OK", cos, cos2)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
