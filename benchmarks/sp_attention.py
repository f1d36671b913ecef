"""Sequence-parallel self-attention of one video / image block, timed across ranks.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29560 \
        benchmarks/sp_attention.py --tokens 32760 --heads 12

Every rank holds ``tokens / world`` tokens of all heads (head dim 128). Two ways to the same
result are timed, each as the max over ranks of the CUDA-event mean after warm-up:

* ``fused``: the exchange inside the kernels (parallel/ulysses.py) - the head-split form when the
  head count divides by the group size, the K / V-to-every-rank form otherwise;
* ``nccl``: the collective form (all-to-all of Q, K, V and of the output, or all-gather of K, V)
  around the plain attention call.

The first call's result of both is compared with fp32 softmax attention on a slice of the queries.
Rank 0 prints one JSON line. Inputs exceed the L2 cache for the default shape (Q, K, V of 32760
tokens x 12 heads are 3 x 100 MB).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=32760, help="tokens of the whole sequence")
    ap.add_argument("--heads", type=int, default=12)
    ap.add_argument("--int8", type=int, default=1)
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--pull", type=int, default=0, help="1: also time the form that reads K / V from their owners (bf16)")
    args = ap.parse_args()

    from hartsyinference_b200 import ops
    from hartsyinference_b200.ops import _native as N
    from hartsyinference_b200.parallel.comm import init_comm
    from hartsyinference_b200.parallel.ulysses import FusedUlyssesAttention

    comm = init_comm()
    rank, world = comm.rank, comm.world
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    torch.cuda.set_device(dev)
    assert args.tokens % world == 0
    s_l, heads, int8 = args.tokens // world, args.heads, bool(args.int8)
    g = torch.Generator(device="cpu").manual_seed(5 + rank)
    q, k, v = ((torch.randn(s_l, heads, 128, generator=g) * (1.0 if i else 0.5)).to(torch.bfloat16).to(dev) for i in range(3))
    split = heads % world == 0

    fused = FusedUlyssesAttention(comm, s_l, heads, dev, int8=int8)

    def run_fused():
        return fused(q, k, v)

    def run_nccl():
        if split:
            qf, kf, vf = (comm.all_to_all(t, split_dim=1, concat_dim=0).contiguous() for t in (q, k, v))
            o = ops.attention(qf, kf, vf, int8=int8)
            return comm.all_to_all(o, split_dim=0, concat_dim=1).reshape(s_l, -1)
        kf = comm.all_gather(k, dim=0)
        vf = comm.all_gather(v, dim=0)
        return ops.attention(q, kf, vf, int8=int8).reshape(s_l, -1)

    def timed(fn) -> float:
        for _ in range(3):
            fn()
        torch.cuda.synchronize(dev)
        comm.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.reps):
            fn()
        b.record()
        torch.cuda.synchronize(dev)
        N.check_status(dev)
        ms = torch.tensor([a.elapsed_time(b) / args.reps], device=dev)
        return _max_over_ranks(comm, ms)

    # numerics on the first 256 local queries against fp32 over the whole sequence
    kf = comm.all_gather(k, dim=0).float()
    vf = comm.all_gather(v, dim=0).float()
    sc = torch.einsum("qhd,khd->hqk", q[:256].float(), kf) * 128 ** -0.5
    want = torch.einsum("hqk,khd->qhd", torch.softmax(sc, -1), vf).reshape(256, -1)
    del kf, vf, sc
    err = {}
    for name, fn in (("fused", run_fused), ("nccl", run_nccl)):
        got = fn()[:256].float()
        err[name] = float((got - want).norm() / want.norm())
    t_fused = timed(run_fused)
    t_nccl = timed(run_nccl)
    t_pull = None
    if args.pull and not int8:
        puller = FusedUlyssesAttention(comm, s_l, heads, dev, pull=True)
        err["pull"] = float((puller(q, k, v)[:256].float() - want).norm() / want.norm())
        t_pull = timed(lambda: puller(q, k, v))
        comm.barrier()
        puller.close()
    flops = 4.0 * args.tokens * args.tokens * heads * 128 / world        # per rank, either form
    if rank == 0:
        print(json.dumps({"case": "sp_attention", "n_gpus": world, "tokens": args.tokens, "heads": heads,
                          "form": "head split" if split else "K / V to every rank", "int8_qk": int8,
                          "fused_ms": t_fused, "nccl_ms": t_nccl, "pull_ms": t_pull, "fused_tflops_per_gpu": flops / t_fused / 1e9,
                          "rel_err_vs_fp32": err, "transport": fused.heap.transport}))
    comm.barrier()
    fused.close()


def _max_over_ranks(comm, t: torch.Tensor) -> float:
    parts = comm.all_gather(t, dim=0)
    return float(parts.max())


if __name__ == "__main__":
    main()
