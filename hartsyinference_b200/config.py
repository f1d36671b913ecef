"""Typed flag registry.

Every runtime switch is declared here once, with a type, a default and a doc string, and is read
from the environment with the single prefix ``B200_``. Nothing else in the package calls
``os.getenv`` for a behaviour switch. The reference scatters 171 ``HARTSY_*`` variables over its
sources and reads most of them ad hoc or through a tri-state helper
(src/HartsyInference.Core/Runtime/EnvSwitch.cs); the same tri-state semantics are kept
(unset -> default, ``0/false/off/no`` -> off, anything else -> on).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Any

_FALSE = {"0", "false", "off", "no", ""}


@dataclass(frozen=True)
class Flag:
    name: str
    type: type
    default: Any
    doc: str

    @property
    def env(self) -> str:
        return "B200_" + self.name.upper()

    def parse(self, raw: str) -> Any:
        if self.type is bool:
            return raw.strip().lower() not in _FALSE
        return self.type(raw)


_REGISTRY: dict[str, Flag] = {}
_OVERRIDES: dict[str, Any] = {}


def declare(name: str, type_: type, default: Any, doc: str) -> Flag:
    if name in _REGISTRY:
        raise ValueError(f"flag {name} declared twice")
    f = Flag(name, type_, default, doc)
    _REGISTRY[name] = f
    return f


def get(name: str) -> Any:
    f = _REGISTRY[name]
    if name in _OVERRIDES:
        return _OVERRIDES[name]
    raw = os.environ.get(f.env)
    if raw is None:
        return f.default
    try:
        return f.parse(raw)
    except ValueError:
        return f.default


def set_override(name: str, value: Any) -> None:
    """Programmatic override (tests, CLI flags); ``None`` removes it."""
    if name not in _REGISTRY:
        raise KeyError(name)
    if value is None:
        _OVERRIDES.pop(name, None)
    else:
        _OVERRIDES[name] = value


def all_flags() -> list[Flag]:
    return sorted(_REGISTRY.values(), key=lambda f: f.name)


def describe() -> str:
    """Human-readable table used by ``--help`` and the docs."""
    rows = [f"{f.env:<34} {f.type.__name__:<6} default={f.default!r:<12} {f.doc}" for f in all_flags()]
    return "\n".join(rows)


# --- declarations -------------------------------------------------------------------------------
declare("log_level", str, "info", "minimum log level: trace, debug, info, warn, error")
declare("profile", bool, False, "accumulate per-op device time (CUDA events) and print a table at exit")
declare("profile_sync", bool, False, "synchronise after every profiled op so host ranges equal device time")
declare("nvtx", bool, False, "emit NVTX ranges around ops and engine phases")
declare("kv_page_size", int, 16, "tokens per KV page")
declare("kv_pool_bytes", int, 0, "KV pool budget in bytes; 0 = size from free device memory")
declare("kv_dtype", str, "bf16", "KV cache dtype: bf16")
declare("cuda_graphs", bool, True, "capture the decode step in CUDA graphs")
declare("max_batch", int, 256, "largest decode batch the scheduler forms")
declare("prefill_chunk", int, 8192, "tokens per prefill chunk")
declare("fused_comm", bool, True, "use the fused compute+collective kernels; off = NCCL baseline")
declare("nvls", bool, True, "allow multimem (in-switch) reductions when the symmetric heap has a multicast mapping")
declare("symm_ipc", bool, False, "map the symmetric heap through CUDA IPC handles even where virtual-memory handles work (no multicast mapping then)")
declare("wait_budget_ms", int, 2000, "budget of every bounded device-side wait")
declare("p2p_disable", bool, False, "never map peer memory; collectives fall back to NCCL")
declare("fp8_linears", bool, True, "quantise eligible linears to 128x128 block-scaled e4m3 at load")
declare("tc_attention", bool, True, "dense non-causal attention with head dim 128 on the tcgen05 kernel instead of the mma.sync one")
declare("fa_attention", bool, True, "dense non-causal head-dim-128 attention on the two-query-tile tcgen05 kernel (S / P / O resident in TMEM); off = the older one-tile tcgen05 kernel")
declare("fused_dit_tp", bool, True, "tensor-parallel DiT: row-parallel linears run as one GEMM + all-reduce + gated-residual kernel; off = GEMM, NCCL all-reduce, gated residual")
declare("fused_dit_sp", bool, True, "tensor-parallel DiT blocks keep activations sharded by token rows between the linears (all-gather -> GEMM, GEMM -> reduce-scatter kernels); off = replicated activations")
declare("fused_cfg_combine", bool, True, "CFG-parallel video pipelines combine the two branches with the peer-memory kernel; off = NCCL all_gather")
declare("fused_ulysses", bool, True, "sequence-parallel attention exchanges heads inside the quantisation / attention kernels (peer stores into the symmetric heap); off = NCCL all-to-all")
declare("mla_fold_q", bool, True, "latent attention on a CUDA device: keep a second query projection with W_uk folded in ([heads * 576, q rank]) and use it for batches of up to 256 rows (one GEMM instead of q_b + per-head absorb); off = always q_b + absorb")
declare("dp_attention", bool, True, "latent-attention MoE models on more than one GPU: decode steps deal the requests over the ranks for the attention block (all heads, replicated attention weights) and exchange tokens around the expert layer; off = tensor-parallel attention over all requests")
declare("fused_dp_exchange", bool, True, "the token exchange of the data-parallel attention layout runs inside the norm / expert-combine kernels over peer memory; off = all_gather / reduce_scatter collectives")
declare("sage_attention", bool, False, "int8 Q K^T (SageAttention: K mean removal, per-row int8 scales, tcgen05 kind::i8) in the dense attention kernel")
declare("decode_attn_stages", int, 2, "depth of the paged decode attention kernel's K/V staging ring: 3 (two CTAs per SM at head dim 128) or 2 (three CTAs per SM)")
declare("cluster_splitk", bool, False, "reduce the K splits of small GEMMs through distributed shared memory of a thread-block cluster instead of a second kernel")
declare("splitk_second_kernel", bool, True, "sum the K splits of a fully split small GEMM with a second, machine-wide kernel (on) or inside the GEMM by the last CTA to arrive at each tile (off)")
declare("kernels_lib", str, "", "path of another build of libb200_kernels.so to load instead of the in-tree one")
declare("pdl", bool, True, "launch GEMMs with programmatic dependent launch so that weight tiles are requested while the preceding kernel still runs")
declare("fp8_scales", str, "ue8m0", "block-scale format of fp8 linears: ue8m0 (power-of-two scales applied by the tensor core) or fp32 (promoted per K block by the epilogue warps)")
declare("gguf_resident", bool, False, "keep Q8_0 / Q4_K GGUF linears as quantised blocks on the device (integer-dot GEMV at decode) instead of dequantising at load")
declare("low_vram", str, "auto", "auto: stream transformer blocks from pinned host memory only when the weights do not fit; on: always stream what can be streamed; off: never")
declare("model_cache_dir", str, "~/.hartsyinference/models", "where resolved checkpoints are cached")
declare("same_gpu_concurrent", bool, False, "allow two requests to share one device slot")
declare("assert_ambient", bool, False, "debug: verify every op runs on the device its tensors live on")
declare("step_cache_threshold", float, 0.0, "first-block-cache relative-L1 threshold; 0 disables")
