"""Profiling support: NVTX ranges, a per-label device-time table, a profiler capture window and
roofline arithmetic against the measured peaks.

Mirrors the reference's ``NvtxRange`` + built-in per-op profiler (``HARTSY_PROFILE``,
``HARTSY_PROFILE_SYNC``; src/HartsyInference.Cuda/Profiling/NvtxRange.cs:33-67) and
``CudaProfilerControl.Window`` (src/HartsyInference.Cuda/Profiling/CudaProfilerControl.cs:22-39),
with CUDA events instead of host ticks so that the table shows device time.
"""
from __future__ import annotations

import contextlib
import json
import os
from collections import defaultdict
from pathlib import Path
from typing import Optional

import torch

from .. import config

_table: dict[str, list] = defaultdict(lambda: [0, 0.0])     # label -> [calls, ms]
_pending: list[tuple[str, torch.cuda.Event, torch.cuda.Event]] = []


@contextlib.contextmanager
def op_range(label: str):
    """NVTX range (``B200_NVTX=1``) and/or device-time accounting (``B200_PROFILE=1``)."""
    use_nvtx = config.get("nvtx") and torch.cuda.is_available()
    prof = config.get("profile") and torch.cuda.is_available()
    if prof and torch.cuda.is_current_stream_capturing():
        prof = False          # timing events recorded into a CUDA graph cannot be read back
    if use_nvtx:
        torch.cuda.nvtx.range_push(label)
    if prof:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
    try:
        yield
    finally:
        if prof:
            b.record()
            if config.get("profile_sync"):
                b.synchronize()
                e = _table[label]
                e[0] += 1
                e[1] += a.elapsed_time(b)
            else:
                _pending.append((label, a, b))
        if use_nvtx:
            torch.cuda.nvtx.range_pop()


def active() -> bool:
    """True when either flag asks for ranges (checked by the op wrappers before they pay for one)."""
    return bool(config.get("profile") or config.get("nvtx"))


def traced(label: str):
    """Decorator: run the function inside ``op_range(label)`` when profiling or NVTX is on."""
    def wrap(fn):
        import functools

        @functools.wraps(fn)
        def inner(*a, **kw):
            if not active():
                return fn(*a, **kw)
            with op_range(label):
                return fn(*a, **kw)
        return inner
    return wrap


def _drain() -> None:
    if _pending:
        torch.cuda.synchronize()
        for label, a, b in _pending:
            e = _table[label]
            e[0] += 1
            e[1] += a.elapsed_time(b)
        _pending.clear()


def reset_profile() -> None:
    _drain()
    _table.clear()


def dump_profile() -> str:
    _drain()
    total = sum(v[1] for v in _table.values()) or 1.0
    rows = sorted(_table.items(), key=lambda kv: -kv[1][1])
    lines = [f"{'op':<32}{'calls':>8}{'ms':>12}{'share':>8}"]
    lines += [f"{k:<32}{v[0]:>8}{v[1]:>12.3f}{100 * v[1] / total:>7.1f}%" for k, v in rows]
    return "\n".join(lines)


@contextlib.contextmanager
def capture_window():
    """cudaProfilerStart/Stop around a region, for ``ncu --profile-from-start off``."""
    if torch.cuda.is_available():
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
    try:
        yield
    finally:
        if torch.cuda.is_available():
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()


# ---------------------------------------------------------------------------------------------
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def measured_peaks(path: Optional[str] = None) -> dict:
    """Roofline denominators: the measured copy bandwidth and cuBLAS bf16 throughput of this
    machine pool when the file exists next to the package root, else the documented fallback."""
    cand = [path] if path else []
    root = Path(__file__).resolve().parents[2]
    cand += [os.environ.get("B200_MEASURED_PEAKS"), str(root / "MEASURED_PEAKS.json")]
    for c in cand:
        if c and Path(c).exists():
            d = json.loads(Path(c).read_text())
            d["source"] = "measured"
            return d
    return dict(FALLBACK_PEAKS)


def roofline(flops: float, bytes_: float, ms: float, peaks: Optional[dict] = None, fp8: bool = False) -> dict:
    """Achieved throughput and its fraction of the measured peak for one kernel launch."""
    p = peaks or measured_peaks()
    tf = flops / ms / 1e9
    gbs = bytes_ / ms / 1e6
    peak_tf = p["bf16_tflops"] * (2.0 if fp8 else 1.0)
    t_compute = flops / (peak_tf * 1e9)
    t_memory = bytes_ / (p["hbm_gbs"] * 1e6)
    bound = "compute" if t_compute > t_memory else "memory"
    return {"tflops": tf, "gbs": gbs, "frac_compute": tf / peak_tf, "frac_memory": gbs / p["hbm_gbs"],
            "bound": bound, "frac_of_roofline": max(t_compute, t_memory) / ms, "peaks": p["source"]}
