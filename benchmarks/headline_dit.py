"""DiT headline workloads of ``bench.py``: Flux-Dev 1024 x 1024 (tensor parallel over N GPUs) and
Wan2.1-14B 81 frames x 720 x 1280 (Ulysses sequence parallel, plus the CFG branch pair once two or
more GPUs are used), random-init weights of the named architecture, synthetic text embeddings.

Each returns the JSON-ready dict of one benchmark line. Two numbers come out of the same timed
steps of one ``pipeline.denoise`` call (the public denoise API): ``value`` from the CUDA events the
pipeline records around every step (max over ranks), ``e2e`` from host wall time around the steps,
which every step copies that step's timestep from pinned host memory and reads the step's latents
back to pinned host memory through the pipeline's per-step callback.

Before the timed run, on more than one GPU, a two-block slice of the same architecture is run in
the parallel layout and on rank 0 alone; the cosine between the two predictions is reported as
``parity``.
"""
from __future__ import annotations

import time
from dataclasses import replace

import torch


def _cos(a: torch.Tensor, b: torch.Tensor) -> float:
    return float(torch.nn.functional.cosine_similarity(a.float().reshape(1, -1), b.float().reshape(1, -1)).item())


class _StepIO:
    """Per-step callback: reads the step's latents back into pinned host memory (what a preview
    consumer does) and stamps host time, so the e2e figure contains a device -> host read per step."""

    def __init__(self):
        self.buf = None
        self.stamps = []
        self.d2h_bytes = 0

    def __call__(self, preview):
        z = preview.latents
        if self.buf is None or self.buf.numel() != z.numel():
            self.buf = torch.empty(z.shape, dtype=z.dtype, pin_memory=True)
        self.buf.copy_(z, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.d2h_bytes = z.numel() * z.element_size()
        self.stamps.append(time.perf_counter())


def _finish(pipe, io: _StepIO, warmup: int, steps: int, comm, dev, ctx_bytes: int):
    ms = pipe.last_step_ms[warmup:warmup + steps]
    wall = (io.stamps[warmup + steps - 1] - io.stamps[warmup - 1]) * 1e3
    t = torch.tensor([sum(ms), wall], device=dev, dtype=torch.float64)
    if comm.world > 1:
        import torch.distributed as dist
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, wall_ms = t.tolist()
    e2e = {"value": wall_ms / steps / 1e3, "unit": "s/step", "ms_per_step": wall_ms / steps,
           "h2d_bytes_per_step": pipe.h2d_bytes_per_step + ctx_bytes // (warmup + steps),
           "d2h_bytes_per_step": io.d2h_bytes}
    return dev_ms / steps, e2e


# ------------------------------------------------------------------------------------------ Flux
def flux_parity(comm, dev, fp8: bool) -> dict:
    from hartsyinference_b200.models.dit import flux as F
    from hartsyinference_b200.parallel.comm import SingleComm
    cfg = replace(F.FLUX_DEV, num_double_blocks=1, num_single_blocks=1)
    g = torch.Generator().manual_seed(11)
    S = 256
    x = (torch.randn(1, S, cfg.in_channels, generator=g) * 0.5).to(torch.bfloat16).to(dev)
    ctx = torch.randn(1, 192, cfg.context_dim, generator=g).to(torch.bfloat16).to(dev)
    pooled = torch.randn(1, cfg.pooled_dim, generator=g).to(torch.bfloat16).to(dev)
    from hartsyinference_b200.pipelines.flux import flux_ids
    img_ids, txt_ids = flux_ids(16, 16, 192, dev)
    sigma, gvec = torch.tensor([0.7], device=dev), torch.tensor([3.5], device=dev)
    tp = F.FluxTransformer(cfg, dev, comm=comm, fp8=fp8, seed=5)
    got = tp.forward(x, ctx, sigma, pooled, img_ids, txt_ids, gvec).float()
    path = getattr(tp, "comm_path", "nccl")
    tp.close()
    del tp
    cos = 1.0
    if comm.rank == 0:
        one = F.FluxTransformer(cfg, dev, comm=SingleComm(), fp8=fp8, seed=5)
        cos = _cos(got, one.forward(x, ctx, sigma, pooled, img_ids, txt_ids, gvec))
        del one
    c = torch.tensor([cos], device=dev)
    if comm.world > 1:
        comm.broadcast(c, 0)
    torch.cuda.empty_cache()
    return {"ok": bool(c.item() > 0.99), "cos": float(c.item()), "what": f"1 double + 1 single block, 256 image + 192 text tokens, tp{comm.world} vs tp1",
            "path": path}


def run_flux(args, comm, dev, sampler) -> dict:
    from hartsyinference_b200.models.dit import flux as F
    from hartsyinference_b200.pipelines.flux import FluxComponents, FluxPipeline
    fp8 = not args.bf16
    cfg = F.FLUX_DEV
    invalid = []
    if args.layers:
        cfg = replace(cfg, num_double_blocks=args.layers, num_single_blocks=2 * args.layers)
        invalid.append(f"layers={args.layers}")
    parity = flux_parity(comm, dev, fp8) if comm.world > 1 else None
    t0 = time.perf_counter()
    tr = F.FluxTransformer(cfg, dev, comm=comm, fp8=fp8)
    torch.cuda.synchronize()
    t_load = time.perf_counter() - t0
    pipe = FluxPipeline(FluxComponents(tr))
    g = torch.Generator().manual_seed(0)
    ctx = torch.randn(512, cfg.context_dim, generator=g).pin_memory()
    pooled = torch.randn(cfg.pooled_dim, generator=g).pin_memory()
    io = _StepIO()
    steps, warmup = args.steps, max(args.warmup, 1)
    comm.barrier()
    torch.cuda.synchronize()
    if comm.rank == 0:
        sampler.start()
    pipe.denoise(ctx, pooled, 1024, 1024, warmup + steps, 3.5, 0, None, 1.0, io)
    torch.cuda.synchronize()
    comm.barrier()
    clocks = sampler.stop() if comm.rank == 0 else None
    ms_step, e2e = _finish(pipe, io, warmup, steps, comm, dev, ctx.numel() * 4 + pooled.numel() * 4)
    from hartsyinference_b200.ops import _native as N
    N.check_status(dev)
    comm_path = getattr(tr, "comm_path", "nccl") if comm.world > 1 else "none"
    tr.close()
    S, H = 4096 + 512, cfg.hidden_size
    lin = cfg.num_double_blocks * (2 * S * H * (3 * H + H + 2 * cfg.mlp_dim)) + \
        cfg.num_single_blocks * (2 * S * H * (3 * H + cfg.mlp_dim) + 2 * S * (H + cfg.mlp_dim) * H)
    att = (cfg.num_double_blocks + cfg.num_single_blocks) * 4 * S * S * H
    return {
        "metric": "DiT s/step (Flux-Dev-architecture 12B, 1024x1024 = 4096 image + 512 text tokens, fp8 block-scaled linears, TP=N, guidance 3.5)",
        "value": ms_step / 1e3, "unit": "s/step", "n_gpus": comm.world, "steps": steps, "warmup": warmup,
        "ms_per_step": ms_step, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16 activations, fp8-e4m3 linears (128x128 / 1x128 block scales)" if fp8 else "bf16",
        "data": "synthetic: random-init weights, N(0,1) text embeddings and latents",
        "config": {"model": "flux-dev", "global_batch": 1, "seq_len": S, "parallelism": f"tp{comm.world}",
                   "denoise_steps_of_the_workload": 20,
                   "l2": "inputs larger than L2 (12 GB of weights read per step)", "invalid_debug_overrides": invalid,
                   "comm_path": comm_path},
        "e2e": e2e, "gpu_launches": N.launch_count, "clocks": clocks, "parity": parity, "load_s": t_load,
        "flops_per_step": lin + att, "tflops_per_gpu": (lin + att) / (ms_step / 1e3) / 1e12 / comm.world,
        "weight_bytes_per_gpu": tr.weight_bytes(),
    }


# ------------------------------------------------------------------------------------------- Wan
def _wan_groups(comm):
    """Layout on N GPUs: 1 GPU runs both CFG branches in turn; N >= 2 pairs two groups of N / 2
    GPUs (conditional / unconditional), each a Ulysses group. Returns (sp_comm, cfg_comm)."""
    n, r = comm.world, comm.rank
    if n == 1:
        return None, None
    half = n // 2
    # every rank takes part in the creation of every group and keeps the two it belongs to
    groups = [comm.subgroup(list(range(0, half))), comm.subgroup(list(range(half, n)))] if half > 1 else [None, None]
    pairs = [comm.subgroup([i, i + half]) for i in range(half)]
    sp = groups[0 if r < half else 1]
    return sp, pairs[r % half]


def wan_parity(comm, dev, fp8: bool) -> dict:
    from hartsyinference_b200.models.dit import wan as W
    cfg = replace(W.WAN_14B, num_layers=2)
    g = torch.Generator().manual_seed(13)
    lat = (torch.randn(cfg.in_channels, 2, 16, 16, generator=g) * 0.5).to(torch.bfloat16).to(dev)   # 2 x 8 x 8 = 128 tokens
    text = torch.randn(cfg.text_len, cfg.text_dim, generator=g).to(dev)
    t = torch.tensor(500.0, device=dev)
    sp = W.WanTransformer(cfg, dev, sp_comm=comm, fp8=fp8, seed=7)
    got = sp.forward(lat, t, sp.encode_text(text)).float()
    path = sp.exchange_path
    sp.close()
    del sp
    cos = 1.0
    if comm.rank == 0:
        one = W.WanTransformer(cfg, dev, fp8=fp8, seed=7)
        cos = _cos(got, one.forward(lat, t, one.encode_text(text)))
        del one
    c = torch.tensor([cos], device=dev)
    comm.broadcast(c, 0)
    torch.cuda.empty_cache()
    return {"ok": bool(c.item() > 0.99), "cos": float(c.item()), "what": f"2 blocks, 128 tokens, sp{comm.world} vs sp1",
            "path": path}


def run_wan(args, comm, dev, sampler) -> dict:
    from hartsyinference_b200.models.dit import wan as W
    from hartsyinference_b200.pipelines.wan import WanComponents, WanPipeline
    fp8 = not args.bf16
    cfg = W.WAN_14B
    invalid = []
    if args.layers:
        cfg = replace(cfg, num_layers=args.layers)
        invalid.append(f"layers={args.layers}")
    sp_comm, cfg_comm = _wan_groups(comm)
    parity = wan_parity(sp_comm, dev, fp8) if (sp_comm is not None and sp_comm.world > 1) else None
    t0 = time.perf_counter()
    tr = W.WanTransformer(cfg, dev, sp_comm=sp_comm, fp8=fp8)
    torch.cuda.synchronize()
    t_load = time.perf_counter() - t0
    pipe = WanPipeline(WanComponents(tr), cfg_comm=cfg_comm)
    g = torch.Generator().manual_seed(0)
    ctx = torch.randn(cfg.text_len, cfg.text_dim, generator=g).pin_memory()
    neg = torch.randn(cfg.text_len, cfg.text_dim, generator=g).pin_memory()
    frames, h, w = 81, 720, 1280
    io = _StepIO()
    steps, warmup = args.steps, max(args.warmup, 1)
    comm.barrier()
    torch.cuda.synchronize()
    if comm.rank == 0:
        sampler.start()
    pipe.denoise(ctx, neg, frames, h, w, warmup + steps, 5.0, 0, "unipc", on_step=io)
    torch.cuda.synchronize()
    comm.barrier()
    clocks = sampler.stop() if comm.rank == 0 else None
    ms_step, e2e = _finish(pipe, io, warmup, steps, comm, dev, 2 * ctx.numel() * 4)
    from hartsyinference_b200.ops import _native as N
    N.check_status(dev)
    exchange = tr.exchange_path
    tr.close()
    S, H = 21 * 45 * 80, cfg.hidden_size
    lin = cfg.num_layers * (2 * S * H * (4 * H + 2 * H + 2 * cfg.ffn_size))
    att = cfg.num_layers * (4 * S * S * H + 4 * S * cfg.text_len * H)
    flops = 2 * (lin + att)
    spw = sp_comm.world if sp_comm is not None else 1
    par = f"sp{spw}" + ("+cfg2" if cfg_comm is not None else " (both CFG branches in turn)")
    return {
        "metric": "DiT s/step (Wan2.1-14B-architecture, 81 frames 720x1280 = 75600 tokens, both CFG branches, Ulysses SP + CFG-parallel over N GPUs)",
        "value": ms_step / 1e3, "unit": "s/step", "n_gpus": comm.world, "steps": steps, "warmup": warmup,
        "ms_per_step": ms_step, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16 activations and attention, fp8-e4m3 linears (128x128 / 1x128 block scales)" if fp8 else "bf16",
        "data": "synthetic: random-init weights, N(0,1) text embeddings and latents",
        "config": {"model": "wan2.1-14b", "global_batch": 1, "seq_len": S, "parallelism": par,
                   "denoise_steps_of_the_workload": 50, "scheduler": "unipc", "cfg_scale": 5.0,
                   "attention": "bf16 tcgen05 flash attention",
                   "l2": "inputs larger than L2 (activations of 75600 tokens x 5120 alone are 774 MB)",
                   "invalid_debug_overrides": invalid,
                   "comm_path": exchange + (f"; CFG pair: {getattr(pipe, 'cfg_path', 'all-gather of the two velocity fields (NCCL)')}" if cfg_comm is not None else "")},
        "e2e": e2e, "gpu_launches": N.launch_count, "clocks": clocks, "parity": parity, "load_s": t_load,
        "flops_per_step": flops, "tflops_per_gpu": flops / (ms_step / 1e3) / 1e12 / comm.world,
        "weight_bytes_per_gpu": tr.weight_bytes(),
    }
