"""Op namespace of the engine.

One function per op; CUDA tensors go to the hand-written sm_100a kernels in
``libb200_kernels.so`` (and fail loudly if that library is missing), CPU tensors go to the fp32
PyTorch statements in :mod:`.reference`. There is no backend interface and no fallback ladder:
the reference's ``IBackend`` (src/HartsyInference.Core/Backends/IBackend.cs, ~150 ops with CPU
default bodies) collapses into this module plus ``torch.Tensor``.
"""
from .core import (  # noqa: F401
    Fp8Act,
    GgufWeight,
    Int8Weight,
    LinearWeight,
    argmax,
    attention,
    attn_decode,
    attn_paged_biased,
    attn_prefill_paged,
    causal_conv3d,
    cfg_euler_step,
    colbatched_linear,
    dit_qkv,
    embedding,
    fill_random_,
    fp8_mx,
    gated_residual,
    glu,
    gguf_linear,
    int8_linear,
    grouped_linear,
    grouped_linear_dynamic,
    moe_block_capacity,
    moe_dispatch_dynamic,
    moe_capacity,
    moe_combine,
    moe_dispatch,
    moe_route,
    linear,
    mla_attn,
    mla_prep,
    cfg_renorm_euler_step,
    cfg_rownorm_euler_step,
    lincomb,
    msda,
    norm,
    quant_fp8_act,
    quant_int8_act,
    quant_fp8_weight,
    repetition_penalty_,
    rope_kv,
    sample_tokens,
    selective_scan,
)
from . import reference  # noqa: F401


# Every op entry point runs inside a named range when ``B200_PROFILE`` / ``B200_NVTX`` is set
# (per-op device-time table, NVTX ranges for a timeline tool); with both off the wrapper is one
# flag lookup. (The reference wraps its backend calls the same way: NvtxRange + HARTSY_PROFILE,
# src/HartsyInference.Cuda/Profiling/NvtxRange.cs:33-67.)
def _install_ranges() -> None:
    import sys
    from ..utils.profiling import traced
    from . import core
    mod = sys.modules[__name__]
    for name in ("linear", "norm", "glu", "rope_kv", "attn_decode", "attn_prefill_paged", "attn_paged_biased", "attention",
                 "embedding", "argmax", "quant_fp8_act", "grouped_linear", "grouped_linear_dynamic", "moe_route",
                 "moe_dispatch", "moe_dispatch_dynamic", "moe_combine", "mla_prep", "mla_attn", "colbatched_linear",
                 "dit_qkv", "gated_residual", "cfg_euler_step", "causal_conv3d", "gguf_linear", "selective_scan", "sample_tokens"):
        fn = getattr(core, name, None)
        if fn is None:
            continue
        wrapped = traced(name)(fn)
        setattr(core, name, wrapped)          # internal calls (core.linear -> core.gguf_linear) are traced too
        if hasattr(mod, name):
            setattr(mod, name, wrapped)


_install_ranges()
