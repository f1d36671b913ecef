"""Measure DiT denoise-step time (Flux or Wan) on random-init weights of the named architecture.

    python benchmarks/bench_dit.py --model flux --steps 4 [--gpus-env torchrun]
    torchrun --nproc-per-node N -m benchmarks/bench_dit --model flux --tp N
    torchrun --nproc-per-node N -m benchmarks/bench_dit --model wan --sp N [--frames 81 --height 720 --width 1280]

Prints one JSON line: s/step (device-timed, max over ranks), the FLOP estimate and the fraction of
the measured bf16 peak."""
from __future__ import annotations

import argparse
import json
import os
from dataclasses import replace

import os as _os
import sys as _sys

_sys.path.insert(0, _os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))))

import torch

from hartsyinference_b200.parallel import init_comm
from hartsyinference_b200.utils import profiling


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="flux", choices=["flux", "wan", "wan1.3b"])
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--height", type=int, default=0)
    ap.add_argument("--width", type=int, default=0)
    ap.add_argument("--frames", type=int, default=81)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--bf16", action="store_true")
    ap.add_argument("--cfg", action="store_true", help="two guidance branches per step (sequential on one group)")
    args = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    comm = init_comm()
    fp8 = not args.bf16
    peaks = profiling.measured_peaks()
    if args.model == "flux":
        from hartsyinference_b200.models.dit import flux as F
        from hartsyinference_b200.pipelines.flux import FluxComponents, FluxPipeline
        cfg = F.FLUX_DEV
        if args.layers:
            cfg = replace(cfg, num_double_blocks=args.layers, num_single_blocks=2 * args.layers)
        tr = F.FluxTransformer(cfg, dev, comm=comm, fp8=fp8)
        h, w = args.height or 1024, args.width or 1024
        pipe = FluxPipeline(FluxComponents(tr))
        g = torch.Generator().manual_seed(0)
        ctx, pooled = torch.randn(512, cfg.context_dim, generator=g), torch.randn(cfg.pooled_dim, generator=g)
        neg = (torch.randn(512, cfg.context_dim, generator=g), torch.randn(cfg.pooled_dim, generator=g)) if args.cfg else None
        pipe.denoise(ctx, pooled, h, w, args.warmup + args.steps, 3.5, 0, neg, 2.0 if args.cfg else 1.0)
        ms = pipe.last_step_ms[args.warmup:]
        S = (h // 16) * (w // 16) + 512
        H = cfg.hidden_size
        lin = cfg.num_double_blocks * (2 * S * H * (3 * H + H + 2 * cfg.mlp_dim)) + cfg.num_single_blocks * (2 * S * H * (3 * H + cfg.mlp_dim) + 2 * S * (H + cfg.mlp_dim) * H)
        att = (cfg.num_double_blocks + cfg.num_single_blocks) * 4 * S * S * H
        flops = (lin + att) * (2 if args.cfg else 1)
        name, par = "flux-dev 1024x1024" if (h, w) == (1024, 1024) else f"flux-dev {w}x{h}", f"tp{comm.world}"
    else:
        from hartsyinference_b200.models.dit import wan as W
        from hartsyinference_b200.pipelines.wan import WanComponents, WanPipeline
        cfg = W.WAN_14B if args.model == "wan" else W.WAN_1_3B
        if args.layers:
            cfg = replace(cfg, num_layers=args.layers)
        tr = W.WanTransformer(cfg, dev, sp_comm=comm, fp8=fp8)
        h, w = args.height or 480, args.width or 832
        pipe = WanPipeline(WanComponents(tr))
        g = torch.Generator().manual_seed(0)
        ctx = torch.randn(cfg.text_len, cfg.text_dim, generator=g)
        neg = torch.randn(cfg.text_len, cfg.text_dim, generator=g) if args.cfg else None
        pipe.denoise(ctx, neg, args.frames, h, w, args.warmup + args.steps, 5.0 if args.cfg else 1.0, 0, "unipc")
        ms = pipe.last_step_ms[args.warmup:]
        S = ((args.frames - 1) // 4 + 1) * (h // 16) * (w // 16)
        H = cfg.hidden_size
        lin = cfg.num_layers * (2 * S * H * (4 * H + 2 * H + 2 * cfg.ffn_size))
        att = cfg.num_layers * (4 * S * S * H + 4 * S * cfg.text_len * H)
        flops = (lin + att) * (2 if args.cfg else 1)
        name, par = f"{args.model} {w}x{h}x{args.frames}f ({S} tokens)", f"sp{comm.world}"
    t = torch.tensor([sum(ms) / len(ms)], device=dev, dtype=torch.float64)
    if comm.world > 1:
        import torch.distributed as dist
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if comm.rank == 0:
        s_step = float(t.item()) / 1e3
        tf = flops / s_step / 1e12 / comm.world
        print(json.dumps({"model": name, "parallelism": par, "s_per_step": s_step, "steps": len(ms), "fp8": fp8,
                          "flops_per_step": flops, "tflops_per_gpu": tf,
                          "frac_of_measured_bf16_peak": tf / peaks["bf16_tflops_sustained"], "peaks": peaks["source"],
                          "weight_gib_per_gpu": tr.weight_bytes() / 2 ** 30}))
    if comm.world > 1:
        comm.barrier()
        torch.cuda.synchronize()
        os._exit(0)


if __name__ == "__main__":
    main()
