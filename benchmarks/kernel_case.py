"""Runs ONE kernel on a small, fixed case a few times: the program that profiler captures wrap.

    python benchmarks/kernel_case.py gemm fp8 64 28672 4096
    python benchmarks/kernel_case.py grouped fp8 32 16 4096 7168
    python benchmarks/kernel_case.py attn_decode 64 8 1 128 2304
    python benchmarks/kernel_case.py mla 64 16 2304
    python benchmarks/kernel_case.py attn_dense 4608 8

Inputs are larger than the L2 cache where the op is bandwidth bound but stay far below a few GB,
so a full-metric capture (dozens of replays per launch) ends in about a minute. The status word is
checked at the end and the process exits non-zero if a kernel reported a failed wait.
"""
from __future__ import annotations

import math
import sys

import os as _os
import sys as _sys

_sys.path.insert(0, _os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))))

import torch

from hartsyinference_b200 import ops
from hartsyinference_b200.ops import _native as N


def _gemm(argv):
    fp8 = argv[0] == "fp8"
    m, n, k = (int(v) for v in argv[1:4])
    x = (torch.randn(m, k, device="cuda") * 0.5).to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda") * 0.1).to(torch.bfloat16)
    lw = ops.LinearWeight.from_dense(w, fp8=fp8)
    xin = ops.quant_fp8_act(x) if fp8 else x
    out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
    for _ in range(3):
        ops.linear(xin, lw, out=out)


def _grouped(argv):
    fp8 = argv[0] == "fp8"
    groups, m, n, k = (int(v) for v in argv[1:5])
    x = (torch.randn(groups * m, k, device="cuda") * 0.5).to(torch.bfloat16)
    w = (torch.randn(groups * n, k, device="cuda") * 0.1).to(torch.bfloat16)
    lw = ops.LinearWeight.from_dense(w, fp8=fp8)
    xin = ops.quant_fp8_act(x, tile_rows=m) if fp8 else x
    for _ in range(3):
        ops.grouped_linear(xin, lw, groups)


def _attn_decode(argv):
    seqs, hkv, group, d, ctx = (int(v) for v in argv[:5])
    page = 16
    per = (ctx + page - 1) // page
    pool = seqs * per + 1
    kc = torch.randn(pool, hkv, page, d, device="cuda").to(torch.bfloat16)
    vc = torch.randn(pool, hkv, page, d, device="cuda").to(torch.bfloat16)
    table = (torch.randperm(pool - 1, device="cuda")[:seqs * per] + 1).to(torch.int32).reshape(seqs, per)
    lens = torch.full((seqs,), ctx, dtype=torch.int32, device="cuda")
    q = torch.randn(seqs, hkv * group, d, device="cuda").to(torch.bfloat16)
    for _ in range(3):
        ops.attn_decode(q, kc, vc, table, lens, max_kv_len=ctx)


def _mla(argv):
    rows, heads, ctx = (int(v) for v in argv[:3])
    page = 16
    per = (ctx + page - 1) // page
    pool = rows * per + 1
    cache = (torch.randn(pool, page, 576, device="cuda") * 0.5).to(torch.bfloat16)
    table = (torch.randperm(pool - 1, device="cuda")[:rows * per] + 1).to(torch.int32).reshape(rows, per)
    lens = torch.full((rows,), ctx, dtype=torch.int32, device="cuda")
    q = (torch.randn(rows, heads, 576, device="cuda") * 0.3).to(torch.bfloat16)
    for _ in range(3):
        ops.mla_attn(q, cache, table, lens, 1.0 / math.sqrt(192), max_kv_len=ctx)
    ms = _time_cold(lambda: ops.mla_attn(q, cache, table, lens, 1.0 / math.sqrt(192), max_kv_len=ctx))
    print(f"mla {rows} x {heads} x {ctx}: {ms * 1e3:.1f} us ({rows * ctx * 576 * 2 / ms / 1e9:.2f} TB/s of distinct cache bytes, "
          f"{rows * heads * ctx * (576 + 512) * 2 / ms / 1e9:.0f} TFLOP/s)")


def _time(fn, reps=5):
    """Median device time (ms) of ``fn`` over ``reps`` runs after three warm-up runs (CUDA events)."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        ts.append(e0.elapsed_time(e1))
    return sorted(ts)[len(ts) // 2]


def _time_cold(fn, reps=7):
    """Median device time (ms) of ``fn`` with the L2 cache flushed before every run (a 256 MB buffer is
    rewritten), as weights arrive inside a decode step."""
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    ts = []
    for i in range(reps + 2):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        if i >= 2:
            ts.append(e0.elapsed_time(e1))
    return sorted(ts)[len(ts) // 2]


def _mla_proj(argv):
    """mla_proj TOKENS HEADS: the projections around the latent attention of DeepSeek-V3 (hidden 7168,
    q rank 1536, 128 + 64 query dims, 512 latent, 128 value dims) for TOKENS rows and HEADS heads, each
    timed by itself with a cold L2: q_b (fp8), rotary / cache-write prep, W_uk absorb, W_uv, o (fp8)."""
    t, heads = (int(v) for v in argv[:2])
    dev = "cuda"
    bf = lambda *s_: (torch.randn(*s_, device=dev) * 0.05).to(torch.bfloat16)
    q_b = ops.LinearWeight.from_dense(bf(heads * 192, 1536), fp8=True)
    o_w = ops.LinearWeight.from_dense(bf(7168, heads * 128), fp8=True)
    w_uk, w_uv = bf(heads * 512, 128), bf(heads * 128, 512)
    qa8 = ops.quant_fp8_act(bf(t, 1536))
    q = bf(t, heads * 192)
    q_abs = torch.empty(t, heads, 576, dtype=torch.bfloat16, device=dev)
    lat = bf(t, heads * 512)
    v = torch.empty(t, heads * 128, dtype=torch.bfloat16, device=dev)
    v8 = ops.quant_fp8_act(bf(t, heads * 128))
    kv = bf(t, 576)
    cache = torch.zeros(t + 16, 576, dtype=torch.bfloat16, device=dev)
    pos = torch.arange(t, dtype=torch.int32, device=dev)
    slots = torch.arange(t, dtype=torch.int64, device=dev)
    inv_freq = torch.rand(32, device=dev)
    ones = torch.ones(512, dtype=torch.bfloat16, device=dev)
    q_fold = ops.LinearWeight.from_dense(bf(heads * 576, 1536), fp8=True)
    cases = [
        ("q_b fp8", lambda: ops.linear(qa8, q_b), heads * 192 * 1536),
        ("q_b with W_uk folded in, fp8", lambda: ops.linear(qa8, q_fold), heads * 576 * 1536),
        ("mla_prep", lambda: ops.mla_prep(kv, ones, q, q_abs, cache, pos, slots, inv_freq, heads, 192, 128), t * heads * 192 * 2),
        ("W_uk absorb", lambda: ops.colbatched_linear(q, w_uk, heads, 192, q_abs.view(t, heads * 576), 576), heads * 512 * 128 * 2),
        ("W_uv", lambda: ops.colbatched_linear(lat, w_uv, heads, 512, v, 128), heads * 128 * 512 * 2),
        ("o fp8", lambda: ops.linear(v8, o_w), heads * 128 * 7168),
    ]
    for name, fn, nbytes in cases:
        ms = _time_cold(fn)
        print(f"mla_proj {t} x {heads} {name}: {ms * 1e3:.1f} us ({nbytes / ms / 1e9:.2f} TB/s of weight bytes)")


def _attn_dense(argv):
    """attn_dense TOKENS HEADS [fa|fa8|tc|mma]: dense bidirectional attention, head dim 128; prints
    the device time and TFLOP/s (4 * T^2 * 128 * heads) of the chosen kernel."""
    from hartsyinference_b200 import config
    tokens, heads = (int(v) for v in argv[:2])
    mode = argv[2] if len(argv) > 2 else "fa"
    config.set_override("fa_attention", mode in ("fa", "fa8"))
    config.set_override("tc_attention", mode != "mma")
    q = torch.randn(tokens, heads, 128, device="cuda").to(torch.bfloat16)
    k = torch.randn(tokens, heads, 128, device="cuda").to(torch.bfloat16)
    v = torch.randn(tokens, heads, 128, device="cuda").to(torch.bfloat16)
    ms = _time(lambda: ops.attention(q, k, v, int8=mode == "fa8"))
    print(f"attention {mode}: {tokens} tokens x {heads} heads: {ms:.3f} ms, "
          f"{4.0 * tokens * tokens * 128 * heads / ms / 1e9:.0f} TFLOP/s")


def _gemm_ar(argv):
    """gemm_ar M N K WORLD: the fused GEMM + all-reduce + residual + RMSNorm + fp8-emit kernel for
    rank 0 of WORLD with this GPU standing in for its peers (protocol and row share of that rank, no
    NVLink latency), against GEMM + norm kernels on the same operands."""
    from hartsyinference_b200.parallel.comm import ShardEmulationComm
    from hartsyinference_b200.parallel.fused import FusedRowParallel
    m, n, k, world = (int(v) for v in argv[:4])
    x = (torch.randn(m, k, device="cuda") * 0.5).to(torch.bfloat16)
    lw = ops.LinearWeight.from_dense((torch.randn(n, k, device="cuda") * 0.1).to(torch.bfloat16), fp8=True)
    xq = ops.quant_fp8_act(x)
    res = torch.zeros(m, n, device="cuda", dtype=torch.bfloat16)
    nw = torch.ones(n, device="cuda", dtype=torch.bfloat16)
    f = FusedRowParallel(ShardEmulationComm(world), n, torch.device("cuda", 0), emulate_peers=True)
    t_fused = _time(lambda: f(xq, lw, res=res, norm_w=nw, emit_bf16=False, emit_fp8=True), reps=9)
    t_plain = _time(lambda: ops.norm(ops.linear(xq, lw), nw, residual=res, emit_fp8=True, emit_bf16=False), reps=9)
    t_gemm = _time(lambda: ops.linear(xq, lw), reps=9)
    print(f"gemm_ar {m}x{n}x{k} world {world}: fused {t_fused * 1e3:.1f} us, GEMM + norm {t_plain * 1e3:.1f} us, GEMM {t_gemm * 1e3:.1f} us")
    f.close()


def _gemm_ar_large(argv):
    """gemm_ar_large M N K WORLD: the > 128-token form (GEMM + all-reduce + gated residual in one kernel)
    for rank 0 of WORLD with this GPU standing in for its peers, against GEMM + gated-residual kernels."""
    from hartsyinference_b200.parallel.comm import ShardEmulationComm
    from hartsyinference_b200.parallel.fused import FusedRowParallel
    m, n, k, world = (int(v) for v in argv[:4])
    x = (torch.randn(m, k, device="cuda") * 0.5).to(torch.bfloat16)
    lw = ops.LinearWeight.from_dense((torch.randn(n, k, device="cuda") * 0.1).to(torch.bfloat16), fp8=True)
    xq = ops.quant_fp8_act(x)
    res = torch.zeros(m, n, device="cuda", dtype=torch.bfloat16)
    gate = torch.ones(n, device="cuda", dtype=torch.bfloat16)
    f = FusedRowParallel(ShardEmulationComm(world), n, torch.device("cuda", 0), emulate_peers=True, max_large_tokens=m)
    t_fused = _time(lambda: f.large(xq, lw, res=res, gate=gate, slot=0), reps=9)
    t_plain = _time(lambda: ops.gated_residual(res, ops.linear(xq, lw), gate[None], m), reps=9)
    print(f"gemm_ar_large {m}x{n}x{k} world {world}: fused {t_fused * 1e3:.1f} us, GEMM + gated residual {t_plain * 1e3:.1f} us "
          f"({2.0 * m * n * k / t_fused / 1e9:.0f} TFLOP/s fused)")
    f.close()


def _ag_gemm(argv):
    """ag_gemm M N K: all-gather -> GEMM kernel with one rank (copy into the gather buffer, per-tile
    arrival waits, tile rotation), against the plain GEMM on the same operands."""
    from hartsyinference_b200.parallel.comm import SingleComm
    from hartsyinference_b200.parallel.fused import FusedColumnParallel
    m, n, k = (int(v) for v in argv[:3])
    x = (torch.randn(m, k, device="cuda") * 0.5).to(torch.bfloat16)
    lw = ops.LinearWeight.from_dense((torch.randn(n, k, device="cuda") * 0.1).to(torch.bfloat16), fp8=True)
    xq = ops.quant_fp8_act(x)
    f = FusedColumnParallel(SingleComm(), m, k)
    t_fused = _time(lambda: f(xq, lw, m), reps=9)
    t_plain = _time(lambda: ops.linear(xq, lw), reps=9)
    print(f"ag_gemm {m}x{n}x{k}: fused {t_fused * 1e3:.1f} us, GEMM {t_plain * 1e3:.1f} us")
    f.close()


def _ulysses(argv):
    """ulysses TOKENS HEADS [int8]: the exchange-fused attention with one rank (operand push into the
    heap, segment flags, output store, output wait), against the plain attention call."""
    from hartsyinference_b200.parallel.comm import SingleComm
    from hartsyinference_b200.parallel.ulysses import FusedUlyssesAttention
    tokens, heads = (int(v) for v in argv[:2])
    int8 = len(argv) > 2 and argv[2] == "int8"
    q, k, v = (torch.randn(tokens, heads, 128, device="cuda").to(torch.bfloat16) for _ in range(3))
    f = FusedUlyssesAttention(SingleComm(), tokens, heads, int8=int8)
    t_fused = _time(lambda: f(q, k, v))
    t_plain = _time(lambda: ops.attention(q, k, v, int8=int8))
    print(f"ulysses {tokens} x {heads} {'int8' if int8 else 'bf16'}: exchange + attention {t_fused:.3f} ms, attention alone {t_plain:.3f} ms")
    f.close()


def _allreduce(argv):
    """allreduce M N: the peer-memory all-reduce kernel with one rank (protocol only)."""
    from hartsyinference_b200.parallel.comm import SingleComm
    from hartsyinference_b200.parallel.custom_ar import CustomAllReduce
    m, n = (int(v) for v in argv[:2])
    car = CustomAllReduce(SingleComm(), m * n)
    car.input(m, n).normal_()
    t = _time(lambda: car.reduce(m, n), reps=9)
    print(f"allreduce {m}x{n} one rank: {t * 1e3:.1f} us")
    car.close()


def _sample(argv):
    """sample ROWS VOCAB: the device sampler (temperature 0.8, top-k 50, top-p 0.9)."""
    rows, vocab = (int(v) for v in argv[:2])
    logits = torch.randn(rows, vocab, device="cuda") * 3
    f32 = lambda v: torch.full((rows,), v, dtype=torch.float32, device="cuda")
    args = (f32(0.8), torch.full((rows,), 50, dtype=torch.int32, device="cuda"), f32(0.9), f32(0.0),
            torch.arange(rows, dtype=torch.int64, device="cuda"), torch.zeros(rows, dtype=torch.int64, device="cuda"))
    t = _time(lambda: ops.sample_tokens(logits, *args), reps=9)
    print(f"sample {rows} x {vocab}: {t * 1e3:.1f} us")


def _int8(argv):
    """int8 M N K [GROUP]: W8A8 linear (activation rotation + quantisation kernel, int8 GEMM) against the fp8 linear."""
    m, n, k = (int(v) for v in argv[:3])
    group = int(argv[3]) if len(argv) > 3 else 0
    x = (torch.randn(m, k, device="cuda") * 0.5).to(torch.bfloat16)
    w = torch.randn(n, k, device="cuda") * 0.05
    lw8 = ops.Int8Weight.from_dense(w, None, group)
    lwf = ops.LinearWeight.from_dense(w.to(torch.bfloat16), fp8=True)
    t8 = _time(lambda: ops.linear(x, lw8), reps=9)
    tf = _time(lambda: ops.linear(x, lwf), reps=9)
    print(f"int8 {m}x{n}x{k} group {group}: W8A8 {t8 * 1e3:.1f} us ({2.0 * m * n * k / t8 / 1e9:.0f} TFLOP/s incl. quantisation), "
          f"fp8 {tf * 1e3:.1f} us ({2.0 * m * n * k / tf / 1e9:.0f})")


def _triplane(argv):
    """triplane RES: density / colour field of a TripoSR-sized decoder over a RES^3 lattice in one kernel."""
    from hartsyinference_b200.models.threed.triposr import TRIPOSR, TripoSr
    from dataclasses import replace
    res = int(argv[0])
    cfg = replace(TRIPOSR, depth=0)
    m = TripoSr(cfg, "cuda")
    planes = torch.randn(3, 40, 64, 64, device="cuda")
    t = _time(lambda: m.field(planes, resolution=res))
    pts = res ** 3
    flop = pts * 2.0 * (120 * 64 + 8 * 64 * 64 + 64 * 4)
    print(f"triplane {res}^3 = {pts} points: {t:.2f} ms, {flop / t / 1e9:.1f} TFLOP/s fp32, {pts / t / 1e6:.2f} G points/s")


CASES = {"mla_proj": _mla_proj, "gemm_ar_large": _gemm_ar_large, "ag_gemm": _ag_gemm, "ulysses": _ulysses, "allreduce": _allreduce, "sample": _sample,
         "int8": _int8, "triplane": _triplane,
         "gemm_ar": _gemm_ar, "attn_dense": _attn_dense, "gemm": _gemm, "grouped": _grouped, "attn_decode": _attn_decode, "mla": _mla}


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] not in CASES:
        print(__doc__)
        return 2
    torch.manual_seed(0)
    CASES[argv[0]](argv[1:])
    torch.cuda.synchronize()
    N.check_status()
    print("ok")
    return 0


if __name__ == "__main__":
    sys.exit(main())
