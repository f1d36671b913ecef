"""Per-rank compute time of a tensor / expert parallel layout, measured on ONE GPU.

    python benchmarks/bench_shard.py --preset llama-3-70b --tp 8 --batch 64 --prompt-len 2048
    python benchmarks/bench_shard.py --preset deepseek-v3 --tp 8 --batch 256 --prompt-len 1024

Builds rank 0's shard of the model on a communicator without peers (collectives are no-ops, so
the generated tokens mean nothing), prefills the batch and times decode steps with CUDA events
under CUDA graphs. The result is what one GPU of the group spends per step EXCLUDING the
collectives: a lower bound for the group's step time and the place to look for kernel work. It is
not a substitute for the multi-GPU benchmark (``bench.py --gpus N``).
"""
from __future__ import annotations

import argparse
import json
from dataclasses import replace

import os as _os
import sys as _sys

_sys.path.insert(0, _os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))))

import torch

from hartsyinference_b200.engine import LLMEngine, SamplingParams
from hartsyinference_b200.models.llm import config as C
from hartsyinference_b200.models.llm.transformer import DecoderModel
from hartsyinference_b200.ops import _native as N
from hartsyinference_b200.parallel.comm import ShardEmulationComm


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", default="llama-3-70b")
    ap.add_argument("--tp", type=int, default=8)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt-len", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=24)
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (0 = the preset's)")
    ap.add_argument("--bf16", action="store_true")
    ap.add_argument("--fused", action="store_true",
                    help="run the fused GEMM + all-reduce + norm kernel with this GPU standing in for its peers "
                         "(the rank's full protocol and row share; no NVLink latency)")
    args = ap.parse_args()
    cfg = C.PRESETS[args.preset]
    if args.layers:
        cfg = replace(cfg, num_layers=args.layers)
    comm = ShardEmulationComm(args.tp)
    model = DecoderModel(cfg, "cuda", comm=comm, fp8=not args.bf16)
    model.random_init(0)
    if args.fused:
        from hartsyinference_b200.parallel.fused import FusedRowParallel
        model.fused_rp = FusedRowParallel(comm, cfg.hidden_size, model.device, emulate_peers=True)
    dlen = args.steps + 16
    page = 16
    pps = (args.prompt_len + dlen + page - 1) // page + 1
    eng = LLMEngine(model, num_pages=args.batch * pps + 8, page_size=page, max_batch=args.batch, prefill_chunk=8192,
                    max_model_len=pps * page)
    g = torch.Generator().manual_seed(1)
    for p in torch.randint(0, cfg.vocab_size, (args.batch, args.prompt_len), generator=g).tolist():
        eng.add_request(p, SamplingParams(greedy=True, ignore_eos=True, max_tokens=dlen))
    def failed():
        return [r.error for r in eng.requests.values() if r.error]

    while any(len(r.output) == 0 and not r.finished for r in eng.requests.values()):
        eng.step()
        if failed():
            raise SystemExit(f"a step failed: {failed()[0]}")
    for _ in range(4):
        eng.step()
    torch.cuda.synchronize()
    eng.time_steps = True
    ts = []
    for _ in range(args.steps):
        eng.step()
        ts.append(eng.device_ms_last)
        if failed():
            raise SystemExit(f"a step failed: {failed()[0]}")
    N.check_status()
    ts.sort()
    med = ts[len(ts) // 2]
    print(json.dumps({"preset": args.preset, "emulated_rank_of": args.tp, "fused_row_parallel": bool(args.fused), "layers": cfg.num_layers, "batch": args.batch,
                      "prompt_len": args.prompt_len, "ms_per_step_compute_only": med, "ms_min": ts[0],
                      "us_per_layer": 1000 * med / cfg.num_layers, "launches_per_step": eng.kernel_launches_last,
                      "weight_gib": model.weight_bytes() / 2 ** 30,
                      "tokens_per_s_if_collectives_were_free": args.batch / med * 1e3}))


if __name__ == "__main__":
    main()
