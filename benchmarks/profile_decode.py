"""Profile one decode step of the serving engine.

    python benchmarks/profile_decode.py --preset llama-3-8b --batch 64 --prompt-len 2048

Builds a random-init model, prefills ``batch`` prompts, runs a few decode steps, then runs ONE
eager (graph-free) decode step inside a cudaProfilerStart/Stop window so that
``ncu --profile-from-start off --metrics gpu__time_duration.sum`` lists exactly the kernels of one
step. Without a profiler attached it prints the per-op device-time table instead.
"""
from __future__ import annotations

import argparse
from dataclasses import replace

import os as _os
import sys as _sys

_sys.path.insert(0, _os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))))

import torch

from hartsyinference_b200 import config
from hartsyinference_b200.engine import LLMEngine, SamplingParams
from hartsyinference_b200.models.llm import config as C
from hartsyinference_b200.models.llm.transformer import DecoderModel
from hartsyinference_b200.utils import profiling


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", default="llama-3-8b")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt-len", type=int, default=2048)
    ap.add_argument("--bf16", action="store_true")
    ap.add_argument("--tp-shard", type=int, default=1,
                    help="build rank 0's shard of an N-way tensor-parallel group on one GPU (no peers)")
    ap.add_argument("--fused", action="store_true",
                    help="with --tp-shard: run the fused GEMM + all-reduce + norm kernel with this GPU standing in for its peers")
    ap.add_argument("--dp-attention", action="store_true",
                    help="with --tp-shard on a latent-attention MoE preset: rank 0's work of the data-parallel attention "
                         "layout (batch / N requests x all heads, experts over all rows); the exchange is emulated")
    args = ap.parse_args()
    cfg = C.PRESETS[args.preset]
    if args.layers:
        cfg = replace(cfg, num_layers=args.layers)
    dev = torch.device("cuda", 0)
    comm = None
    if args.tp_shard > 1:   # same per-GPU GEMM / attention shapes as rank 0 of a TP group
        from hartsyinference_b200.parallel.comm import ShardEmulationComm
        comm = ShardEmulationComm(args.tp_shard)
    model = DecoderModel(cfg, dev, comm=comm, fp8=not args.bf16, dp_attention=args.dp_attention)
    model.random_init(0)
    if args.dp_attention and comm is not None:
        from hartsyinference_b200.parallel.dp_attention import CollectiveDpExchange

        class _Peerless:
            """Stands in for the group: a gather repeats this rank's rows, a reduce-scatter keeps its share."""
            rank, world = comm.rank, comm.world

            @staticmethod
            def all_gather(t, dim=0):
                return t.repeat_interleave(comm.world, dim=dim) if dim else t.repeat(comm.world, *([1] * (t.dim() - 1)))

            @staticmethod
            def reduce_scatter(t, dim=0):
                return t.chunk(comm.world, dim=dim)[comm.rank].contiguous()

        model.dp_exchange = CollectiveDpExchange(_Peerless, args.batch, cfg.hidden_size, dev)
        model.comm.all_gather = _Peerless.all_gather        # the final gather of the hidden states
    if args.fused and comm is not None:
        from hartsyinference_b200.parallel.fused import FusedRowParallel
        model.fused_rp = FusedRowParallel(comm, cfg.hidden_size, dev, emulate_peers=True)
    total = args.prompt_len + 64
    pages = (total + 15) // 16 + 1
    eng = LLMEngine(model, num_pages=args.batch * pages + 8, page_size=16, max_batch=args.batch, prefill_chunk=8192,
                    max_model_len=pages * 16, use_cuda_graphs=False)
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, cfg.vocab_size, (args.batch, args.prompt_len), generator=g).tolist()
    for p in prompts:
        eng.add_request(p, SamplingParams(greedy=True, ignore_eos=True, max_tokens=32))
    while any(len(r.output) == 0 for r in eng.requests.values()):
        eng.step()
    for _ in range(3):
        eng.step()
    torch.cuda.synchronize()
    config.set_override("profile", True)
    profiling.reset_profile()
    eng.time_steps = True
    with profiling.capture_window():
        eng.step()
    print(f"decode step device time: {eng.device_ms_last:.3f} ms, launches: {eng.kernel_launches_last}")
    print(profiling.dump_profile())


if __name__ == "__main__":
    main()
