"""Placement and parallelism planners for a uniform NVSwitch box.

``suggest`` picks (tp, sp, ep, cfg, pp, dp) from the model's bytes, its shape and the GPU count,
and logs a ``[ParallelPlan]`` line like the reference's ``ParallelPlanner.Suggest``
(src/HartsyInference.Engine/Placement/ParallelPlanner.cs:40; FitOverhead 1.3 :32). ``llm_split_plan``
/ ``dit_split_plan`` / ``largest_remainder_counts`` / ``validate_placement`` restate the layer-split
planners (PlacementPlanner.cs: LlmSplitPlan:22, DitSplitPlan:145,196, ValidatePlacement:304-392,
LargestRemainderCounts:396) for pipeline (layer / block) sharding.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

from .. import log
from ..parallel.config import ParallelConfig

FIT_OVERHEAD = 1.3          # weights * 1.3 must fit (activations, KV, workspace)
GPU_BYTES = 180 * 10**9


@dataclass(frozen=True)
class ModelShape:
    kind: str                 # "llm" | "moe_llm" | "image_dit" | "video_dit"
    weight_bytes: int
    num_heads: int = 0
    num_kv_heads: int = 0
    ffn_size: int = 0
    hidden_size: int = 0
    num_experts: int = 0
    seq_tokens: int = 0       # DiT: tokens per sample
    true_cfg: bool = False    # two guidance branches per step


def largest_remainder_counts(total: int, ratios: Sequence[float]) -> list[int]:
    """Split ``total`` items proportionally to ``ratios`` (largest-remainder rounding, every share >= 0)."""
    s = float(sum(ratios))
    if s <= 0 or total <= 0:
        return [0] * len(ratios)
    exact = [total * r / s for r in ratios]
    counts = [int(e) for e in exact]
    rest = total - sum(counts)
    order = sorted(range(len(ratios)), key=lambda i: (exact[i] - counts[i], -i), reverse=True)
    for i in order[:rest]:
        counts[i] += 1
    return counts


def llm_split_plan(num_layers: int, devices: int, ratios: Optional[Sequence[float]] = None) -> list[range]:
    """Contiguous layer ranges per pipeline stage."""
    counts = largest_remainder_counts(num_layers, ratios or [1.0] * devices)
    out, start = [], 0
    for c in counts:
        out.append(range(start, start + c))
        start += c
    return out


def dit_split_plan(block_bytes: Sequence[int], devices: int) -> list[range]:
    """Byte-weighted contiguous split of DiT blocks over pipeline stages."""
    total = sum(block_bytes)
    target = total / devices
    out, start, acc = [], 0, 0
    for i, b in enumerate(block_bytes):
        acc += b
        stages_left = devices - len(out) - 1          # stages still to open after the current one
        blocks_left = len(block_bytes) - (i + 1)
        if stages_left > 0 and (acc >= target or blocks_left == stages_left) and blocks_left >= stages_left:
            out.append(range(start, i + 1))
            start, acc = i + 1, 0
    out.append(range(start, len(block_bytes)))
    while len(out) < devices:
        out.append(range(len(block_bytes), len(block_bytes)))
    return out[:devices]


def validate_placement(cfg: ParallelConfig, gpus: int, shape: Optional[ModelShape] = None) -> list[str]:
    """Returns a list of human-readable problems (empty = valid)."""
    errs = []
    need = cfg.tp * cfg.sp * cfg.cfg * cfg.pp * cfg.dp
    if need > gpus:
        errs.append(f"placement needs {need} GPUs, {gpus} available")
    if cfg.cfg not in (1, 2):
        errs.append("cfg parallel degree must be 1 or 2")
    if shape is not None:
        if cfg.tp > 1 and shape.num_heads and shape.num_heads % cfg.tp:
            errs.append(f"{shape.num_heads} heads do not divide by tp={cfg.tp}")
        if cfg.tp > 1 and shape.ffn_size and shape.ffn_size % cfg.tp:
            errs.append(f"ffn {shape.ffn_size} does not divide by tp={cfg.tp}")
        if cfg.sp > 1 and shape.num_heads and shape.num_heads % cfg.sp:
            errs.append(f"{shape.num_heads} heads do not divide by sp={cfg.sp} (Ulysses needs whole heads per rank)")
        if cfg.ep > 1 and shape.num_experts and shape.num_experts % cfg.ep:
            errs.append(f"{shape.num_experts} experts do not divide by ep={cfg.ep}")
        per_gpu = shape.weight_bytes * FIT_OVERHEAD / max(1, cfg.tp * cfg.pp * (cfg.ep if shape.num_experts else 1))
        if per_gpu > GPU_BYTES:
            errs.append(f"{per_gpu / 1e9:.0f} GB per GPU exceeds {GPU_BYTES / 1e9:.0f} GB")
    return errs


def suggest(shape: ModelShape, gpus: int, latency_bound: bool = True) -> ParallelConfig:
    """Choose a parallel layout for ``gpus`` identical NVSwitch-connected B200s."""
    def largest_divisor(n: int, limit: int) -> int:
        for d in range(min(limit, n), 0, -1):
            if n % d == 0 and limit % d == 0:
                return d
        return 1

    if gpus <= 1:
        plan = ParallelConfig()
    elif shape.kind in ("image_dit", "video_dit"):
        cfg = 2 if shape.true_cfg and gpus >= 2 else 1
        rest = gpus // cfg
        if shape.kind == "video_dit" or shape.seq_tokens >= 16384:
            sp = largest_divisor(shape.num_heads or rest, rest)
            plan = ParallelConfig(sp=sp, cfg=cfg, dp=max(1, rest // sp))
        else:
            tp = largest_divisor(shape.num_heads or rest, rest)
            plan = ParallelConfig(tp=tp, cfg=cfg, dp=max(1, rest // tp))
    elif shape.kind == "moe_llm":
        # experts are sharded over the tensor-parallel group (activations replicated, one all-reduce
        # for routed + shared outputs), so ep rides on tp
        g = largest_divisor(shape.num_experts or gpus, gpus)
        if shape.num_heads:
            g = largest_divisor(shape.num_heads, g)
        plan = ParallelConfig(tp=g, ep=g, dp=max(1, gpus // g))
    else:
        fits_one = shape.weight_bytes * FIT_OVERHEAD <= GPU_BYTES
        tp = largest_divisor(shape.num_heads or gpus, gpus)
        if fits_one and not latency_bound:
            plan = ParallelConfig(dp=gpus)           # throughput: replicas
        else:
            plan = ParallelConfig(tp=tp, dp=max(1, gpus // tp))
    problems = validate_placement(plan, gpus, shape)
    if problems:
        log.decision("ParallelPlan", f"suggested {plan.describe()} rejected ({'; '.join(problems)}); using single")
        plan = ParallelConfig()
    log.decision("ParallelPlan", f"{shape.kind} {shape.weight_bytes / 1e9:.1f} GB on {gpus} GPU(s) -> {plan.describe()}")
    return plan


def shape_of_checkpoint(path) -> Optional[ModelShape]:
    """Model shape for :func:`suggest` from a Hugging Face-style directory (``config.json`` + weight
    files) or a single weight file; None when nothing can be read."""
    import json
    from pathlib import Path
    p = Path(path)
    if not p.exists():
        return None
    files = [p] if p.is_file() else [f for f in p.rglob("*") if f.suffix in (".safetensors", ".gguf", ".bin", ".pt")]
    nbytes = sum(f.stat().st_size for f in files)
    cfg = {}
    for cand in ((p / "config.json"), (p / "transformer" / "config.json")) if p.is_dir() else ():
        if cand.exists():
            try:
                cfg = json.loads(cand.read_text())
                break
            except Exception:
                pass
    heads = int(cfg.get("num_attention_heads") or cfg.get("n_head") or 0)
    experts = int(cfg.get("n_routed_experts") or cfg.get("num_local_experts") or cfg.get("num_experts") or 0)
    cls = str(cfg.get("_class_name", "")).lower()
    if "transformer3d" in cls or "wan" in cls:
        kind = "video_dit"
    elif "transformer2d" in cls or "flux" in cls or "sd3" in cls:
        kind = "image_dit"
    else:
        kind = "moe_llm" if experts else "llm"
    return ModelShape(kind=kind, weight_bytes=nbytes, num_heads=heads,
                      num_kv_heads=int(cfg.get("num_key_value_heads") or heads),
                      ffn_size=int(cfg.get("intermediate_size") or 0), hidden_size=int(cfg.get("hidden_size") or 0),
                      num_experts=experts)
