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
    norm,
    quant_fp8_act,
    quant_fp8_weight,
    repetition_penalty_,
    rope_kv,
    selective_scan,
)
from . import reference  # noqa: F401
