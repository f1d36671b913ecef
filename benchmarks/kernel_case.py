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


CASES = {"gemm_ar": _gemm_ar, "attn_dense": _attn_dense, "gemm": _gemm, "grouped": _grouped, "attn_decode": _attn_decode, "mla": _mla}


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
