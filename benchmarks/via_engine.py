"""The headline decode benchmark driven through the public serving API.

``bench.py --via engine`` lands here: an :class:`InferenceEngine` is built for the placement
``tp = number of ranks``, a ``synthetic:<preset>`` model (random-init weights of the named
architecture) is loaded through it, and ``batch`` client threads each stream one request of
``prompt_len`` uniform-random token ids with ``engine.text.stream`` — the call an application makes.
Ranks other than 0 serve as followers (``engine.follow()``), exactly as under ``cli serve``.

Timed region: ``steps`` consecutive iterations of the serving loop, starting ``warmup`` iterations
after the one that finished the last prefill, all of them full decode steps (every request produced
a token). The end-to-end figure is the wall clock on rank 0 between the ends of the first and last
of those iterations, while all client threads are streaming: it contains the scheduler, the
per-step host-to-device copies from pinned memory, the device-to-host read of the sampled tokens
and the hand-off of tokens to the clients. The device-timed figure next to it is the sum of the
CUDA-event times of the same iterations, the maximum over ranks.
"""
from __future__ import annotations

import threading
import time

import torch


def run(args, world: int, rank: int, local_rank: int, sampler, metric: str) -> dict | None:
    from hartsyinference_b200.engine.inference_engine import InferenceEngine
    from hartsyinference_b200.engine.requests import ChunkKind, EngineOptions, ModelSpec, TextRequest
    from hartsyinference_b200.models.llm import config as C
    from hartsyinference_b200.ops import _native as N
    from hartsyinference_b200.parallel.config import ParallelConfig

    cfg = C.PRESETS[args.preset]
    total_len = args.prompt_len + args.decode_len
    opts = EngineOptions(placement=ParallelConfig(tp=world), max_batch=args.batch, max_model_len=total_len + 32,
                         kv_pool_bytes_budget=args.batch * (total_len + 32) * cfg.num_layers * 2 * cfg.kv_size * 2 // world + (64 << 20))
    eng = InferenceEngine(f"cuda:{local_rank}" if torch.cuda.is_available() else "cpu", opts)
    name = f"synthetic:{args.preset}" + (f":layers={args.layers}" if args.layers else "")
    spec = ModelSpec(requested=name)
    def hosted_engine():
        return next(iter(eng.text._models.values())).engine

    def arm():
        e = hosted_engine()
        e.time_steps = True
        e.step_log = []

    def step_log():
        log_r = list(hosted_engine().step_log or [])
        return eng.ranks.gather(log_r) if eng.ranks is not None else [log_r]

    if eng.ranks is not None:
        # the followers must know these before they start following
        eng.ranks.register("bench.arm", arm)
        eng.ranks.register("bench.steplog", step_log)
    if not eng.is_front:
        eng.follow()
        return None

    t0 = time.perf_counter()
    hosted = eng.text._host(spec)
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    t_load = time.perf_counter() - t0
    if eng.ranks is not None:
        eng.ranks.command("bench.arm")
    else:
        arm()
    g = torch.Generator().manual_seed(1234)
    prompts = torch.randint(0, cfg.vocab_size, (args.batch, args.prompt_len), generator=g).tolist()

    def client(i: int) -> None:
        # the full decode length of the workload: requests that finish their prefill early keep
        # decoding while the others are still prefilling, so the steady state (every request
        # decoding) is only reached when each request has tokens left by then
        req = TextRequest(prompt_token_ids=prompts[i], greedy=True, ignore_eos=True, max_tokens=args.decode_len)
        for _ in eng.text.stream(spec, req):
            pass

    threads = [threading.Thread(target=client, args=(i,), daemon=True) for i in range(args.batch)]
    sampler.start()
    w0 = time.perf_counter()
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    clocks = sampler.stop()
    if torch.cuda.is_available():
        N.check_status(torch.device("cuda", local_rank))
    logs = (eng.ranks.command("bench.steplog") if eng.ranks is not None else step_log()) or []
    log0 = logs[0]
    # decode steps: the ones in which every request produced a token
    decode = [e for e in log0 if e[5] == args.batch]
    if len(decode) < args.warmup + args.steps:
        raise RuntimeError(f"only {len(decode)} full decode steps ran; lower --steps")
    first = next(i for i, e in enumerate(log0) if e[5] == args.batch)      # the step that finished the last prefill
    a, b = first + 1 + args.warmup, first + 1 + args.warmup + args.steps
    window = log0[a:b]
    if len(window) < args.steps or not all(e[5] == args.batch for e in window):
        raise RuntimeError("the steady state (every request decoding) lasted fewer steps than asked for; lower --steps or raise --decode-len")
    wall_ms = (window[-1][0] - log0[a - 1][0]) * 1e3
    dev_ms = max(sum(e[1] for e in lg[a:b]) for lg in logs if lg)
    tokens = args.steps * args.batch
    ttft = log0[first][0] - w0
    out = {
        "metric": metric, "value": tokens / (dev_ms / 1e3) if dev_ms > 0 else None, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dev_ms / args.steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None,
        "dtype": "fp8-e4m3 weights+activations (128x128 / 1x128 block scales), bf16 KV and accumulators out",
        "data": "synthetic: random-init weights, uniform-random prompt token ids",
        "config": {"model": args.preset, "global_batch": args.batch, "seq_len": args.prompt_len, "decode_len": args.decode_len,
                   "parallelism": f"tp{world}", "kv_page": opts.kv_page_size, "via": "InferenceEngine.text.stream, one client thread per request",
                   "l2": "inputs larger than L2 (weights + KV read per step >> 126 MB)",
                   "fused_comm": getattr(hosted.llm.model, "fused_rp", None) is not None,
                   "invalid_debug_overrides": [f"layers={args.layers}"] if args.layers else []},
        "e2e": {"value": tokens / (wall_ms / 1e3), "unit": "tokens/s", "ms_per_step": wall_ms / args.steps,
                "h2d_bytes_per_step": sum(e[3] for e in window) // args.steps, "d2h_bytes_per_step": sum(e[4] for e in window) // args.steps,
                "what": "wall clock on rank 0 between the ends of two engine steps of the serving loop, with all client threads streaming"},
        "gpu_launches": sum(e[2] for e in window), "clocks": clocks, "ttft_s": {"batch_first_token_wall": ttft},
        "load_s": t_load,
    }
    eng.close()
    return out
