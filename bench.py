#!/usr/bin/env python
"""Headline benchmark: decode throughput of a Llama-3-70B-architecture model served with fp8
(128x128 block-scaled) weights, tensor-parallel over N GPUs, continuous batching of 64 requests
with 2048-token prompts and paged KV (16-token pages).

    python bench.py --gpus N --steps K --warmup W          (N > 1: launched through torchrun)

The other headline workloads run through ``--preset``: ``deepseek-v3`` (DeepSeek-V3 architecture,
fp8, 256 x (1024 + 128), experts sharded over N = 8 GPUs; decode tok/s), ``flux-dev`` (Flux-Dev
1024 x 1024, TP = N; s/step) and ``wan-14b`` (Wan2.1-14B, 81 frames x 720 x 1280, sequence parallel
+ CFG-parallel over N GPUs; s/step), see ``benchmarks/headline_dit.py``. On more than one GPU every
preset first checks a two-layer slice of its model in the parallel layout against one rank alone
and reports it as ``parity``.

A "step" is one engine decode iteration for the whole batch (64 new tokens). The weights are
random-init tensors of the named architecture and the prompts are uniform-random token ids
(there is no network for checkpoints or datasets). The prompts are really prefilled, so the KV
pool holds 2048+ tokens of context per request while the decode steps are timed.

Two numbers come out of the same K timed steps, both through the public engine API
(``LLMEngine.step``), which every step copies the batch metadata (token ids, positions, KV slots,
block tables, lengths) from pinned host memory to the device and reads the sampled ids back:
  * ``value``      tokens/s from CUDA-event device time of the steps (max over ranks),
  * ``e2e.value``  tokens/s from host wall time around the K steps (max over ranks), i.e. including
                   the scheduler, the host-side batch assembly and the synchronising read-back.
``--impl reference`` reports that the reference cannot run here (it is a .NET solution; no .NET
SDK exists on the build or the GPU machine and it has no Python packaging).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--preset", default="llama-3-70b",
                    choices=["llama-3-70b", "deepseek-v3", "flux-dev", "wan-14b", "llama-3-8b", "qwen2.5-0.5b"],
                    help="workload (the headline is llama-3-70b)")
    ap.add_argument("--batch", type=int, default=0, help="requests (default: 64; deepseek-v3: 256)")
    ap.add_argument("--prompt-len", type=int, default=0, help="prompt tokens (default: 2048; deepseek-v3: 1024)")
    ap.add_argument("--decode-len", type=int, default=0, help="decode tokens (default: 256; deepseek-v3: 128)")
    ap.add_argument("--no-parity", action="store_true", help="skip the multi-GPU parity block")
    ap.add_argument("--layers", type=int, default=0, help="debug only: override the layer count (marks the run invalid)")
    ap.add_argument("--bf16", action="store_true", help="debug only: bf16 weights instead of fp8")
    ap.add_argument("--no-fused-comm", action="store_true", help="NCCL all-reduce instead of the fused kernels")
    ap.add_argument("--force-fused", action="store_true", help="keep the fused kernels even where GEMM + NCCL measures faster")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--via", default="steps", choices=["steps", "engine"],
                    help="steps: drive LLMEngine.step directly (the headline); engine: client threads streaming through "
                         "InferenceEngine.text, followers under engine.follow() (benchmarks/via_engine.py)")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples: list[list[str]] = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        def pump():
            for line in self.proc.stdout:
                self.samples.append([c.strip() for c in line.split(",")])
        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        mhz, mx, reasons = [], None, set()
        for s in self.samples:
            try:
                mhz.append(float(s[1]))
                mx = float(s[2])
                for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7),
                                  ("sw_power_cap", 8)):
                    if s[col].lower().startswith("active"):
                        reasons.add(name)
            except Exception:
                continue
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": mx,
                "reasons": sorted(reasons), "samples": len(mhz)}


def run_reference(args) -> int:
    print(json.dumps({
        "impl": "reference",
        "unavailable": "reference is a C#/.NET solution without Python packaging (pip: no setup.py/pyproject.toml) "
                       "and no .NET SDK exists on this machine, so its CUDA backend cannot be built or run",
    }))
    return 0


def main() -> int:
    args = parse_args()
    if args.impl == "reference":
        return run_reference(args)

    import torch
    from hartsyinference_b200 import config as hconfig
    from hartsyinference_b200 import log
    from hartsyinference_b200.engine import LLMEngine, SamplingParams
    from hartsyinference_b200.models.llm import config as C
    from hartsyinference_b200.models.llm.transformer import DecoderModel
    from hartsyinference_b200.parallel import init_comm
    from hartsyinference_b200.ops import _native as N

    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    rank = int(os.environ.get("RANK", "0"))
    if world != args.gpus:
        if args.gpus > 1 and world == 1:
            # re-launch under torchrun when called directly with --gpus N
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
                   "--master-addr", "127.0.0.1", "--master-port", os.environ.get("MASTER_PORT", "29517"),
                   os.path.abspath(__file__)] + sys.argv[1:]
            return subprocess.call(cmd)
    if args.via == "engine":
        if args.preset in ("flux-dev", "wan-14b"):
            print(json.dumps({"unavailable": "--via engine covers the text presets"}))
            return 0
        dsv3 = args.preset == "deepseek-v3"
        args.batch = args.batch or (256 if dsv3 else 64)
        args.prompt_len = args.prompt_len or (1024 if dsv3 else 2048)
        args.decode_len = args.decode_len or (128 if dsv3 else 256)
        if torch.cuda.is_available():
            torch.cuda.set_device(local_rank)
        sys.path.insert(0, os.path.join(ROOT, "benchmarks"))
        import via_engine
        out = via_engine.run(args, world, rank, local_rank, ClockSampler(local_rank), _metric_name(args))
        if out is not None:
            print(json.dumps(out))
        sys.stdout.flush()
        if world > 1:
            os._exit(0)
        return 0
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    comm = init_comm()
    if rank != 0:
        import logging
        log.logger.setLevel(logging.WARNING)
    sys.path.insert(0, os.path.join(ROOT, "benchmarks"))
    if args.preset in ("flux-dev", "wan-14b"):
        import headline_dit
        fn = headline_dit.run_flux if args.preset == "flux-dev" else headline_dit.run_wan
        out = fn(args, comm, device, ClockSampler(local_rank))
        if rank == 0:
            print(json.dumps(out))
        return _leave(comm, world)
    dsv3 = args.preset == "deepseek-v3"
    args.batch = args.batch or (256 if dsv3 else 64)
    args.prompt_len = args.prompt_len or (1024 if dsv3 else 2048)
    args.decode_len = args.decode_len or (128 if dsv3 else 256)

    cfg = C.PRESETS[args.preset]
    invalid = []
    if args.layers:
        from dataclasses import replace
        cfg = replace(cfg, num_layers=args.layers)
        invalid.append(f"layers={args.layers}")
    if args.bf16:
        invalid.append("bf16 weights")
    need = _weight_bytes_estimate(cfg, world, fp8=not args.bf16)
    total_mem = torch.cuda.get_device_properties(device).total_memory
    if need > 0.8 * total_mem:
        if rank == 0:
            print(json.dumps({"metric": _metric_name(args), "n_gpus": world, "value": None,
                              "unavailable": f"{need / 2**30:.0f} GiB of weights per GPU at {world} GPU(s) do not fit "
                                             f"{total_mem / 2**30:.0f} GiB of device memory",
                              "config": {"model": args.preset, "parallelism": f"tp{world}"}}))
        return _leave(comm, world)
    parity = None
    if world > 1 and not args.no_parity:
        import llm_parity
        def _enable(m):
            if args.no_fused_comm:
                return False
            from hartsyinference_b200.parallel.fused import enable_fused_tp
            return enable_fused_tp(m, comm)
        parity = llm_parity.run(cfg, comm, device, not args.bf16, _enable,
                                dp_attention=cfg.mla is not None and bool(hconfig.get("dp_attention")),
                                dp_fused=False if args.no_fused_comm else None)
        if rank == 0:
            log.info(f"[Bench] parity {parity}")
    t0 = time.perf_counter()
    # latent-attention MoE models: decode steps deal the requests over the ranks for the attention block
    dp_attn = world > 1 and cfg.mla is not None and bool(hconfig.get("dp_attention")) and args.batch % world == 0
    model = DecoderModel(cfg, device, comm=comm, fp8=not args.bf16, dp_attention=dp_attn)
    model.random_init(seed=0)
    dp_fused = False
    if dp_attn:
        from hartsyinference_b200.parallel.dp_attention import enable_dp_attention
        dp_fused = enable_dp_attention(model, comm, max_rows=args.batch, fused=False if args.no_fused_comm else None)
    fused = False
    if world > 1 and not args.no_fused_comm:
        try:
            from hartsyinference_b200.parallel.fused import enable_fused_tp
            fused = enable_fused_tp(model, comm, max_tokens=max(args.batch, 128),
                                    autotune_tokens=0 if args.force_fused else args.batch, large_tokens=8192)
        except Exception as e:  # keep the run alive on NCCL, but say so
            log.warn(f"[Collective] fused TP kernels unavailable ({type(e).__name__}: {e}); using NCCL")
    torch.cuda.synchronize()
    t_load = time.perf_counter() - t0

    total_len = args.prompt_len + args.decode_len
    page = 16
    pages_per_seq = (total_len + page - 1) // page + 1
    eng = LLMEngine(model, num_pages=args.batch * pages_per_seq + 8, page_size=page, max_batch=args.batch,
                    prefill_chunk=8192, max_model_len=pages_per_seq * page, use_cuda_graphs=not args.no_graphs)
    g = torch.Generator().manual_seed(1234)      # same prompts on every rank
    prompts = torch.randint(0, cfg.vocab_size, (args.batch, args.prompt_len), generator=g).tolist()
    params = SamplingParams(greedy=True, ignore_eos=True, max_tokens=args.decode_len)
    for p in prompts:
        eng.add_request(p, params)

    # ---- prefill (untimed for the headline; reported as TTFT of the whole batch)
    comm.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    first_token_times = []
    while any(len(r.output) == 0 for r in eng.requests.values()):
        eng.step()
    torch.cuda.synchronize()
    t_prefill = time.perf_counter() - t0
    ttft = sorted(r.t_first_token - r.t_submit for r in eng.requests.values())
    N.check_status(device)

    steps_possible = args.decode_len - 3 - args.warmup
    steps = min(args.steps, steps_possible)
    for _ in range(args.warmup):
        eng.step()
    torch.cuda.synchronize()
    peer_ar = getattr(model, "custom_ar", None) is not None
    multimem = bool(getattr(getattr(model, "fused_rp", None) or getattr(model, "custom_ar", None), "use_mc", False))
    if fused or peer_ar or dp_fused:
        # A bounded wait of the peer-memory kernels that gave up on any rank means the peer protocol
        # did not work on this machine: fall back to NCCL on every rank rather than time garbage.
        bad = torch.tensor([int(N.state(device).status[0].item() != 0)], device=device)
        import torch.distributed as dist
        dist.all_reduce(bad, op=dist.ReduceOp.MAX)
        if int(bad.item()) != 0:
            log.warn("[Collective] peer-memory kernels reported a wait timeout; falling back to NCCL")
            N.state(device).reset_after_fault()
            from hartsyinference_b200.parallel.fused import disable_fused_tp
            disable_fused_tp(model, comm)
            if dp_fused:
                from hartsyinference_b200.parallel.dp_attention import enable_dp_attention
                model.dp_exchange.close()
                dp_fused = enable_dp_attention(model, comm, max_rows=args.batch, fused=False)
            peer_ar = False
            eng._graphs.clear()
            fused = False
            for _ in range(2):
                eng.step()
            torch.cuda.synchronize()
    comm.barrier()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    eng.time_steps = True
    dev_ms = 0.0
    launches = 0
    h2d = d2h = 0
    comm.barrier()
    torch.cuda.synchronize()
    w0 = time.perf_counter()
    for _ in range(steps):
        ev = eng.step()
        dev_ms += eng.device_ms_last
        launches += eng.kernel_launches_last
        h2d += eng.h2d_bytes_last
        d2h += eng.d2h_bytes_last
        assert len(ev) == args.batch
    torch.cuda.synchronize()
    comm.barrier()
    wall_ms = (time.perf_counter() - w0) * 1e3
    clocks = sampler.stop() if rank == 0 else None
    N.check_status(device)

    t = torch.tensor([dev_ms, wall_ms], dtype=torch.float64, device=device)
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, wall_ms = t.tolist()
    tokens = steps * args.batch
    if rank == 0:
        out = {
            "metric": _metric_name(args),
            "value": tokens / (dev_ms / 1e3),
            "unit": "tokens/s",
            "n_gpus": world,
            "steps": steps,
            "warmup": args.warmup,
            "ms_per_step": dev_ms / steps,
            "higher_is_better": True,
            "scaling": "strong",
            "vs_baseline": None,
            "dtype": "fp8-e4m3 weights+activations (128x128 / 1x128 block scales), bf16 KV and accumulators out",
            "data": "synthetic: random-init weights, uniform-random prompt token ids",
            "config": {"model": args.preset, "global_batch": args.batch, "seq_len": args.prompt_len,
                       "decode_len": args.decode_len, "parallelism": f"tp{world}", "kv_page": page,
                       "l2": "inputs larger than L2 (weights + KV read per step >> 126 MB)",
                       "cuda_graphs": not args.no_graphs, "fused_comm": fused, "multimem": multimem,
                       "comm_path": "fused GEMM+all-reduce" if fused else "peer-memory all-reduce kernel" if peer_ar else ("nccl" if world > 1 else "none"),
                       "attention_layout": (f"data parallel at decode: {args.batch // world} requests x all heads per rank, tokens exchanged around "
                                            f"the expert layer {'inside the norm / combine kernels (peer stores)' if dp_fused else 'with all_gather / reduce_scatter'}; "
                                            "prefill tensor parallel") if model.dp_exchange is not None else "tensor parallel",
                       "invalid_debug_overrides": invalid},
            "e2e": {"value": tokens / (wall_ms / 1e3), "unit": "tokens/s", "ms_per_step": wall_ms / steps,
                    "h2d_bytes_per_step": h2d // steps, "d2h_bytes_per_step": d2h // steps},
            "gpu_launches": launches,
            "clocks": clocks,
            "parity": parity,
            "ttft_s": {"batch_prefill_wall": t_prefill, "median": ttft[len(ttft) // 2], "max": ttft[-1]},
            "load_s": t_load,
            "weight_bytes_per_gpu": model.weight_bytes(),
        }
        print(json.dumps(out))
    if world > 1:
        eng._graphs.clear()
        from hartsyinference_b200.parallel.fused import disable_fused_tp
        disable_fused_tp(model, comm)
        if model.dp_exchange is not None:
            torch.cuda.synchronize()
            comm.barrier()
            model.dp_exchange.close()
    return _leave(comm, world)


def _leave(comm, world: int) -> int:
    """Every rank has taken its memory out of the multicast object and unmapped its peers before
    any rank leaves. NCCL communicators that were captured into CUDA graphs can block in their
    teardown; the result is already printed, so leave without running it."""
    if world > 1:
        import torch
        comm.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)
    return 0


def _metric_name(args) -> str:
    if args.preset == "deepseek-v3":
        return (f"decode tok/s (DeepSeek-V3-architecture MoE, fp8 128x128 block-scaled weights, experts sharded over N GPUs, "
                f"{args.batch} x ({args.prompt_len} prompt + {args.decode_len} decode), MLA latent KV)")
    name = {"llama-3-70b": "Llama-3-70B"}.get(args.preset, args.preset)
    return (f"decode tok/s ({name}-architecture, fp8 128x128 block-scaled weights, TP=N, "
            f"{args.batch} x ({args.prompt_len} prompt + {args.decode_len} decode), paged KV)")


def _weight_bytes_estimate(cfg, world: int, fp8: bool) -> int:
    """Bytes of weights one rank will hold (linears fp8 or bf16, embeddings bf16)."""
    H, L = cfg.hidden_size, cfg.num_layers
    per = 1 if fp8 else 2
    if cfg.mla is not None:
        m = cfg.mla
        attn = H * (m.q_lora_rank or 0) + (m.q_lora_rank or H) * cfg.num_heads * (m.qk_nope_head_dim + m.qk_rope_head_dim) // world \
            + H * (m.kv_lora_rank + m.qk_rope_head_dim) * 2 // per + cfg.num_heads * m.kv_lora_rank * (m.qk_nope_head_dim + m.v_head_dim) * 2 // per // world \
            + H * cfg.num_heads * m.v_head_dim // world
    else:
        attn = H * (cfg.q_size + 2 * cfg.kv_size) // world + H * cfg.q_size // world
    dense = 3 * H * cfg.ffn_size // world
    total = 0
    for li in range(L):
        moe = cfg.moe is not None and cfg.moe.num_experts > 0 and li >= cfg.moe.first_dense_layers
        if moe:
            total += attn + 3 * H * cfg.moe.expert_ffn * cfg.moe.num_experts // world \
                + 3 * H * cfg.moe.shared_ffn * cfg.moe.num_shared_experts // world
        else:
            total += attn + dense
    emb = cfg.vocab_size * H * 2 * (1 if cfg.tie_embeddings else 1 + 1 / world)
    if cfg.mla is not None and world > 1:
        # the data-parallel attention layout also keeps the attention weights of all heads on every rank
        m = cfg.mla
        dq = m.qk_nope_head_dim + m.qk_rope_head_dim
        full = (m.q_lora_rank or H) * cfg.num_heads * dq + H * cfg.num_heads * m.v_head_dim \
            + cfg.num_heads * m.kv_lora_rank * (m.qk_nope_head_dim + m.v_head_dim) * 2 // per
        total += L * full
    return int(total * per + emb)


if __name__ == "__main__":
    sys.exit(main())
