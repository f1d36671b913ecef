"""Int8 weight formats with per-output-row scales ("int8_tensorwise"), with and without the ConvRot
Hadamard rotation.

A ConvRot checkpoint stores ``W @ H^T`` row-quantised to int8, where ``H`` is the normalised regular
Hadamard matrix ``kron(h4, ..., h4)`` applied per contiguous group of ``G`` input features (``G`` a
power of four). ``H`` is symmetric and orthogonal, so the consumer either rotates the activation by
``H`` at run time and multiplies in int8, ``(x H)(W H^T)^T = x W^T`` (:func:`ops.linear` with an
:class:`~hartsyinference_b200.ops.Int8Weight`: rotation + quantisation kernel, then the tcgen05 int8
GEMM), or un-rotates the weight once at load (:func:`dequant_to_bf16`).

The rotation is a radix-4 butterfly, ``log4(G)`` stages of the 4x4 seed
``h4 = 1/2 [[1,1,1,-1],[1,1,-1,1],[1,-1,1,1],[-1,1,1,1]]``: every output of a stage is half of (the sum
of its four inputs minus twice the mirrored input).

Reference: src/HartsyInference.Core/Tensors/Int8ConvRotCodec.cs (BuildHadamard:23, DequantToBf16:62,
ApplyRotation:124), src/HartsyInference.Cuda/Kernels/dequant/convrot.cu.
"""
from __future__ import annotations

from typing import Optional

import torch


def is_valid_group(size: int) -> bool:
    """A power of four, at least 4."""
    if size < 4 or size & (size - 1):
        return False
    return (size.bit_length() - 1) % 2 == 0


def rotate(t: torch.Tensor, group: int) -> torch.Tensor:
    """``t @ blockdiag(H, ..., H)`` along the last dim (fp32 math), ``H`` of size ``group``."""
    if group <= 1:
        return t.float()
    if not is_valid_group(group) or t.shape[-1] % group != 0:
        raise ValueError(f"ConvRot group size {group} must be a power of four dividing {t.shape[-1]}")
    x = t.float().reshape(*t.shape[:-1], t.shape[-1] // group, group)
    stride = 1
    while stride < group:
        # digits of the index at this stage: [..., blocks, 4, stride]
        y = x.reshape(*x.shape[:-1], group // (4 * stride), 4, stride)
        s = y.sum(dim=-2, keepdim=True)
        x = (0.5 * (s - 2.0 * y.flip(-2))).reshape(*x.shape[:-1], group)
        stride *= 4
    return x.reshape(t.shape)


def hadamard(size: int) -> torch.Tensor:
    """The matrix itself ([size, size] fp32): the rotation of the identity."""
    return rotate(torch.eye(size), size)


def quantize_weight(w: torch.Tensor, group: int = 0) -> tuple[torch.Tensor, torch.Tensor]:
    """bf16 / fp32 ``w`` [N, K] -> (int8 [N, K] of ``W H^T`` (``W`` itself when ``group`` is 0), fp32 row
    scales [N])."""
    r = rotate(w, group) if group > 1 else w.float()
    amax = r.abs().amax(dim=1)
    scale = torch.where(amax > 0, amax / 127.0, torch.ones_like(amax))
    q = torch.clamp(torch.round(r / scale[:, None]), -127, 127).to(torch.int8)
    return q, scale.float()


def dequant_to_bf16(q: torch.Tensor, row_scale: torch.Tensor, group: int = 0) -> torch.Tensor:
    """The plain bf16 weight of an int8 (ConvRot) tensor: scale, then un-rotate (``H`` is its own
    inverse). ``row_scale`` holds one value per row or a single per-tensor value."""
    s = row_scale.float().reshape(-1)
    w = q.float() * (s[:, None] if s.numel() == q.shape[0] else s[0])
    return (rotate(w, group) if group > 1 else w).to(torch.bfloat16)


def quantize_activation(x: torch.Tensor, group: int = 0, inv_smooth: Optional[torch.Tensor] = None) -> tuple[torch.Tensor, torch.Tensor]:
    """fp32 statement of the activation side: smooth, rotate, quantise per row. -> (int8 [M, K], fp32 [M])."""
    v = x.float()
    if inv_smooth is not None:
        v = v * inv_smooth.float()
    v = rotate(v, group) if group > 1 else v
    amax = v.abs().amax(dim=1)
    scale = torch.where(amax > 0, amax / 127.0, torch.ones_like(amax))
    inv = torch.where(amax > 0, 127.0 / amax, torch.zeros_like(amax))
    q = torch.clamp(torch.round(v * inv[:, None]), -127, 127).to(torch.int8)
    return q, scale.float()
