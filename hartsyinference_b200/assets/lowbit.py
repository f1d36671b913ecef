"""Low-bit weight codecs: MXFP4 / MXFP8 (OCP microscaling: 32-element blocks with a power-of-two
E8M0 scale), NVFP4 (16-element blocks with an E4M3 scale under one fp32 tensor scale), NF4
(16-level normal-float table, 64-element absmax blocks), and the 128 x 4 blocked scale layout the
tensor-core block-scaled MMA reads.

Checkpoints stored in these formats are decoded at load (to bf16, or re-quantised to the fp8
block-scaled layout the GEMM runs); the encoders exist for conversion and for tests.

Reference: src/HartsyInference.ModelAssets/ low-bit codecs (Mxfp4, Mxfp8, Nf4, Nvfp4,
BlockScale/BlockScaleSwizzle.cs), src/HartsyInference.Core quant side info.
"""
from __future__ import annotations

import torch

# E2M1 magnitudes by code (sign is bit 3)
E2M1 = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
E2M1_MAX = 6.0
E4M3_MAX = 448.0

# bitsandbytes' NF4 levels: quantiles of N(0, 1) normalised to [-1, 1], with an exact zero
NF4 = torch.tensor([-1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635,
                    -0.18477343022823334, -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725,
                    0.24611230194568634, 0.33791524171829224, 0.44070982933044434, 0.5626170039176941,
                    0.7229568362236023, 1.0])


# ------------------------------------------------------------------------------------ fp4 / e8m0
def e2m1_encode(x: torch.Tensor) -> torch.Tensor:
    """fp32 -> 4-bit E2M1 codes (uint8 0..15), round to nearest with ties to the even code."""
    mag = x.abs().float().clamp(max=E2M1_MAX)
    table = E2M1.to(x.device)
    # boundaries between neighbouring magnitudes; a tie goes to the code whose mantissa bit is 0
    mid = (table[1:] + table[:-1]) / 2
    idx = torch.bucketize(mag, mid, right=False)             # mag == mid -> lower code
    tie = (mag[..., None] == mid).any(-1)
    lower_is_even = (idx % 2) == 0
    idx = torch.where(tie & ~lower_is_even, idx + 1, idx)
    return (idx.to(torch.uint8) | ((x < 0).to(torch.uint8) << 3)).to(torch.uint8)


def e2m1_decode(code: torch.Tensor) -> torch.Tensor:
    mag = E2M1.to(code.device)[(code & 7).long()]
    return torch.where((code & 8) != 0, -mag, mag)


def pack_nibbles(code: torch.Tensor) -> torch.Tensor:
    """[..., 2n] codes -> [..., n] bytes, element 2i in the low nibble."""
    return (code[..., 0::2] | (code[..., 1::2] << 4)).to(torch.uint8)


def unpack_nibbles(packed: torch.Tensor) -> torch.Tensor:
    out = torch.stack([packed & 0xF, packed >> 4], -1)
    return out.reshape(*packed.shape[:-1], packed.shape[-1] * 2)


def e8m0_from_amax(amax: torch.Tensor, elem_max: float) -> torch.Tensor:
    """Smallest power of two s (as a biased E8M0 byte) with amax / s <= elem_max."""
    ratio = (amax.float() / elem_max).clamp_min(2.0 ** -127)
    e = torch.ceil(torch.log2(ratio)).clamp(-127, 127)
    return (e + 127).to(torch.uint8)


def e8m0_decode(b: torch.Tensor) -> torch.Tensor:
    return torch.pow(2.0, b.float() - 127.0)


# ------------------------------------------------------------------------------------ MXFP4 / MXFP8
def mxfp4_quantize(w: torch.Tensor, block: int = 32) -> tuple[torch.Tensor, torch.Tensor]:
    """[rows, k] -> (packed codes [rows, k / 2] uint8, scales [rows, k / block] E8M0 bytes)."""
    rows, k = w.shape
    assert k % block == 0
    x = w.float().reshape(rows, k // block, block)
    sc = e8m0_from_amax(x.abs().amax(-1), E2M1_MAX)
    q = e2m1_encode(x / e8m0_decode(sc)[..., None])
    return pack_nibbles(q.reshape(rows, k)), sc


def mxfp4_dequantize(packed: torch.Tensor, scales: torch.Tensor, block: int = 32) -> torch.Tensor:
    rows = packed.shape[0]
    v = e2m1_decode(unpack_nibbles(packed)).reshape(rows, -1, block)
    return (v * e8m0_decode(scales)[..., None]).reshape(rows, -1)


def mxfp8_quantize(w: torch.Tensor, block: int = 32) -> tuple[torch.Tensor, torch.Tensor]:
    """[rows, k] -> (E4M3 values [rows, k] as float8_e4m3fn, scales [rows, k / block] E8M0 bytes)."""
    rows, k = w.shape
    assert k % block == 0
    x = w.float().reshape(rows, k // block, block)
    sc = e8m0_from_amax(x.abs().amax(-1), E4M3_MAX)
    q = (x / e8m0_decode(sc)[..., None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return q.reshape(rows, k), sc


def mxfp8_dequantize(q: torch.Tensor, scales: torch.Tensor, block: int = 32) -> torch.Tensor:
    rows = q.shape[0]
    return (q.float().reshape(rows, -1, block) * e8m0_decode(scales)[..., None]).reshape(rows, -1)


# ------------------------------------------------------------------------------------ NVFP4
def nvfp4_quantize(w: torch.Tensor, block: int = 16) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """[rows, k] -> (packed codes [rows, k / 2], block scales [rows, k / block] float8_e4m3fn,
    tensor scale fp32 scalar). value = code * block_scale * tensor_scale."""
    rows, k = w.shape
    assert k % block == 0
    x = w.float().reshape(rows, k // block, block)
    amax = x.abs().amax(-1)
    tensor_scale = (amax.max() / (E2M1_MAX * E4M3_MAX)).clamp_min(1e-30)
    bs = (amax / E2M1_MAX / tensor_scale).clamp(max=E4M3_MAX).to(torch.float8_e4m3fn)
    denom = (bs.float() * tensor_scale).clamp_min(1e-30)
    q = e2m1_encode(x / denom[..., None])
    return pack_nibbles(q.reshape(rows, k)), bs, tensor_scale.reshape(())


def nvfp4_dequantize(packed: torch.Tensor, block_scales: torch.Tensor, tensor_scale: torch.Tensor, block: int = 16) -> torch.Tensor:
    rows = packed.shape[0]
    v = e2m1_decode(unpack_nibbles(packed)).reshape(rows, -1, block)
    return (v * block_scales.float()[..., None] * tensor_scale.float()).reshape(rows, -1)


# ------------------------------------------------------------------------------------ NF4
def nf4_quantize(w: torch.Tensor, block: int = 64) -> tuple[torch.Tensor, torch.Tensor]:
    """Flattened tensor -> (packed codes [n / 2] uint8 with the first element in the high nibble, the
    bitsandbytes order; absmax [n / block] fp32)."""
    x = w.float().flatten()
    assert x.numel() % block == 0
    xb = x.reshape(-1, block)
    absmax = xb.abs().amax(-1).clamp_min(1e-30)
    n = xb / absmax[:, None]
    code = (n[..., None] - NF4.to(x.device)).abs().argmin(-1).to(torch.uint8).flatten()
    return ((code[0::2] << 4) | code[1::2]).to(torch.uint8), absmax


def nf4_dequantize(packed: torch.Tensor, absmax: torch.Tensor, shape, block: int = 64) -> torch.Tensor:
    code = torch.stack([packed >> 4, packed & 0xF], -1).flatten().long()
    v = NF4.to(packed.device)[code].reshape(-1, block) * absmax.float()[:, None]
    return v.reshape(shape)


# ------------------------------------------------------------------------------------ blocked scales
def swizzle_block_scales(scales: torch.Tensor) -> torch.Tensor:
    """Row-major block scales [rows, cols] (one byte each) -> the blocked layout of the block-scaled
    tensor-core MMA: tiles of 128 rows x 4 columns stored as 512 bytes where row r, column c sits at
    (r % 32) * 16 + (r // 32) * 4 + c; tiles ordered row tile major. Rows and columns are zero-padded
    to multiples of 128 and 4."""
    assert scales.element_size() == 1
    rows, cols = scales.shape
    rp, cp = -(-rows // 128) * 128, -(-cols // 4) * 4
    s = torch.zeros(rp, cp, dtype=torch.uint8, device=scales.device)
    s[:rows, :cols] = scales.view(torch.uint8)
    t = s.reshape(rp // 128, 4, 32, cp // 4, 4)          # [row tile, r // 32, r % 32, col tile, c]
    return t.permute(0, 3, 2, 1, 4).contiguous().reshape(-1)


def unswizzle_block_scales(blocked: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    rp, cp = -(-rows // 128) * 128, -(-cols // 4) * 4
    t = blocked.reshape(rp // 128, cp // 4, 32, 4, 4).permute(0, 3, 2, 1, 4)
    return t.reshape(rp, cp)[:rows, :cols].contiguous()


# ------------------------------------------------------------------------------------ checkpoints
def dequantizing_get(get):
    """Wrap a checkpoint's ``get(name)`` so that quantised linears read as bf16 ``<module>.weight``:

    * fp8 block-scaled (DeepSeek-V3 / Qwen3-FP8): ``weight`` float8_e4m3 + ``weight_scale_inv``
      [ceil(out / 128), ceil(in / 128)] fp32
    * fp8 per-tensor / per-channel: ``weight`` float8 + ``weight_scale``
    * NVFP4 (ModelOpt): ``weight`` uint8 [out, in / 2] + ``weight_scale`` e4m3 [out, in / 16] + ``weight_scale_2``
    * NVFP4 (compressed-tensors): ``weight_packed`` + ``weight_scale`` + ``weight_global_scale`` (divides)
    * MXFP4 (GPT-OSS style): ``<module>_blocks`` uint8 [..., k / 32, 16] + ``<module>_scales`` E8M0 [..., k / 32]
    * NF4 (bitsandbytes): ``weight`` uint8 + ``weight.absmax`` (+ ``weight.quant_map``)

    Anything else passes through untouched."""
    def g(name: str):
        t = get(name)
        if not name.endswith(".weight"):
            return t
        stem = name[: -len(".weight")]
        if t is None:
            packed = get(stem + ".weight_packed")
            if packed is not None:
                gs = get(stem + ".weight_global_scale")
                ts = (1.0 / gs.float().reshape(())) if gs is not None else torch.tensor(1.0)
                return nvfp4_dequantize(packed, get(stem + ".weight_scale"), ts).to(torch.bfloat16)
            blocks = get(stem + "_blocks")
            if blocks is not None:
                sc = get(stem + "_scales")
                flat = blocks.reshape(-1, blocks.shape[-2] * blocks.shape[-1])
                w = mxfp4_dequantize(flat, sc.reshape(flat.shape[0], -1))
                return w.reshape(*blocks.shape[:-2], -1).to(torch.bfloat16)
            return None
        if t.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
            inv = get(stem + ".weight_scale_inv")
            if inv is not None:
                o, i = t.shape
                s = inv.float().repeat_interleave(128, 0)[:o].repeat_interleave(128, 1)[:, :i]
                return (t.float() * s).to(torch.bfloat16)
            sc = get(stem + ".weight_scale")
            if sc is not None:
                sc = sc.float()
                return (t.float() * (sc if sc.dim() == 0 else sc.reshape(-1, 1))).to(torch.bfloat16)
            return t.to(torch.bfloat16)
        if t.dtype == torch.uint8:
            absmax = get(name + ".absmax")
            if absmax is not None:
                qmap = get(name + ".quant_map")
                shape_t = get(name + ".shape")
                n = t.numel() * 2
                code = torch.stack([t.flatten() >> 4, t.flatten() & 0xF], -1).flatten().long()
                table = qmap.float() if qmap is not None else NF4
                v = table[code].reshape(-1, n // absmax.numel()) * absmax.float().flatten()[:, None]
                return (v.reshape(tuple(int(x) for x in shape_t)) if shape_t is not None else v.flatten()).to(torch.bfloat16)
            bs = get(stem + ".weight_scale")
            if bs is not None and bs.dtype == torch.float8_e4m3fn:
                ts = get(stem + ".weight_scale_2")
                return nvfp4_dequantize(t, bs, ts.float().reshape(()) if ts is not None else torch.tensor(1.0)).to(torch.bfloat16)
        return t
    return g
