"""Python entry points of the fused ops (see the package docstring for the dispatch rule)."""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass
from typing import Optional

import torch

from . import _native as N
from . import reference as R

_ACT = {None: 0, "none": 0, "gelu_tanh": 1, "silu": 2}


def fp8_mx() -> bool:
    """True when fp8 linears use UE8M0 (power-of-two) block scales applied by the tensor core
    (config flag ``fp8_scales``), False for fp32 scales promoted by the epilogue."""
    from .. import config
    return config.get("fp8_scales") == "ue8m0"


def _tc_attention() -> bool:
    from .. import config
    return bool(config.get("tc_attention"))


def _alloc_sf(rows: int, k: int, tile_rows: int, device) -> torch.Tensor:
    """Blocked scale-factor array for ``rows`` x ``k`` e4m3 values (see reference.pack_sf). Bytes of
    K blocks past the end of K must be finite (they meet zero data), so a ragged last group is
    zero-filled; rows past the end only feed output rows that are never stored."""
    tiles, kg = (rows + tile_rows - 1) // tile_rows, (k + 511) // 512
    if k % 512:
        return torch.zeros(tiles, kg, 128, dtype=torch.int32, device=device)
    return torch.empty(tiles, kg, 128, dtype=torch.int32, device=device)


@dataclass
class Fp8Act:
    """e4m3 activations [M, K] (uint8 storage) with 1x128 scales: fp32 ``scale`` [M, K/128], or
    (device, UE8M0 mode) the blocked scale-factor array ``sf`` covering ``tile_rows`` rows per block."""
    data: torch.Tensor
    scale: Optional[torch.Tensor]
    sf: Optional[torch.Tensor] = None
    tile_rows: int = 128

    @property
    def shape(self):
        return self.data.shape

    def scales_fp32(self) -> torch.Tensor:
        """The scales as fp32 [M, K/128] whichever way they are stored."""
        if self.scale is not None:
            return self.scale
        m, k = self.data.shape
        return R.unpack_sf(self.sf, m, k // 128, self.tile_rows)


@dataclass
class LinearWeight:
    """Weight of a linear layer, [N, K] K-major. bf16, or e4m3 bytes with 128x128 block scales
    [ceil(N/128), K/128]."""
    weight: torch.Tensor
    scale: Optional[torch.Tensor] = None
    bias: Optional[torch.Tensor] = None
    sf: Optional[torch.Tensor] = None       # UE8M0 mode: blocked scale factors built from ``scale``

    @property
    def is_fp8(self) -> bool:
        return self.scale is not None

    @property
    def is_mx(self) -> bool:
        return self.sf is not None

    def host_f32(self) -> torch.Tensor:
        """fp32 copy of a host-resident bf16 weight, made once: the CPU path multiplies in fp32 and
        would otherwise widen the whole matrix on every call."""
        c = self.__dict__.get("_host_f32")
        if c is None or c.shape != self.weight.shape:
            c = self.weight.float()
            self.__dict__["_host_f32"] = c
        return c

    @staticmethod
    def from_quantized(q: torch.Tensor, scale: torch.Tensor, bias: Optional[torch.Tensor] = None) -> "LinearWeight":
        """e4m3 bytes [N, K] + block scales [ceil(N/128), K/128]. In UE8M0 mode the scales must be
        powers of two (they are rounded to the nearest one) and the blocked array is built here."""
        if fp8_mx():
            scale = torch.exp2(torch.log2(scale.float()).round())
            sf = R.pack_sf(scale.repeat_interleave(128, dim=0)[:((q.shape[0] + 127) // 128) * 128], 128)
            return LinearWeight(q, scale.contiguous(), bias, sf.contiguous())
        return LinearWeight(q, scale, bias)

    @property
    def out_features(self) -> int:
        return self.weight.shape[0]

    @property
    def in_features(self) -> int:
        return self.weight.shape[1]

    def nbytes(self) -> int:
        n = self.weight.numel() * self.weight.element_size()
        if self.scale is not None:
            n += self.scale.numel() * 4
        if self.sf is not None:
            n += self.sf.numel() * 4
        if self.bias is not None:
            n += self.bias.numel() * self.bias.element_size()
        return n

    @staticmethod
    def from_dense(w: torch.Tensor, bias: Optional[torch.Tensor] = None, fp8: bool = False) -> "LinearWeight":
        w = w.to(torch.bfloat16).contiguous()
        if fp8 and w.shape[1] % 128 == 0:
            q, s = quant_fp8_weight(w)
            return LinearWeight.from_quantized(q, s, None if bias is None else bias.to(torch.bfloat16))
        return LinearWeight(w, None, None if bias is None else bias.to(torch.bfloat16))


@dataclass
class Int8Weight:
    """W8A8 linear weight: int8 [N, K] with one fp32 scale per output row, optionally stored rotated
    (ConvRot: ``W H^T`` per group of ``convrot_group`` input features, see assets/int8_convrot.py) and
    with per-input-channel SmoothQuant factors ``inv_smooth`` [K] applied to the activations."""
    weight: torch.Tensor
    row_scale: torch.Tensor
    bias: Optional[torch.Tensor] = None
    convrot_group: int = 0
    inv_smooth: Optional[torch.Tensor] = None

    @staticmethod
    def from_dense(w: torch.Tensor, bias: Optional[torch.Tensor] = None, convrot_group: int = 0) -> "Int8Weight":
        from ..assets.int8_convrot import quantize_weight
        q, s = quantize_weight(w.float().cpu(), convrot_group)
        return Int8Weight(q.to(w.device).contiguous(), s.to(w.device), None if bias is None else bias.to(torch.bfloat16),
                          convrot_group)

    def nbytes(self) -> int:
        return self.weight.numel() + self.row_scale.numel() * 4 + (0 if self.bias is None else self.bias.numel() * 2)

    @property
    def out_features(self) -> int:
        return self.weight.shape[0]

    @property
    def in_features(self) -> int:
        return self.weight.shape[1]


def quant_int8_act(x: torch.Tensor, convrot_group: int = 0, inv_smooth: Optional[torch.Tensor] = None):
    """bf16 [M, K] -> (int8 [M, K], fp32 row scales [M]) after the optional SmoothQuant factors and the
    ConvRot rotation; one kernel on the device."""
    if not x.is_cuda:
        from ..assets.int8_convrot import quantize_activation
        return quantize_activation(x, convrot_group, inv_smooth)
    m, k = x.shape
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1
    q = torch.empty(m, k, dtype=torch.int8, device=x.device)
    sc = torch.empty(m, dtype=torch.float32, device=x.device)
    N.check(N.lib().b200_quant_int8_rows(x.data_ptr(), q.data_ptr(), sc.data_ptr(), N.ptr(inv_smooth), m, k, x.stride(0), k,
                                         int(convrot_group), N.stream()), "b200_quant_int8_rows")
    return q, sc


def int8_linear(x: torch.Tensor, w: Int8Weight, act: Optional[str] = None, gate: Optional[torch.Tensor] = None,
                residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = residual + gate * act((x H) (W H^T)^T + bias) with int8 operands and s32 accumulation on the
    tensor core (tcgen05 kind::i8); the two scale vectors are applied by the GEMM epilogue. Replaces the
    reference's cublasLt int8 GEMM + dequant pass (src/HartsyInference.Cuda/Kernels/dequant/w8a8.cu,
    int8_mma_gemm.cu:221)."""
    q, sc = quant_int8_act(x, w.convrot_group, w.inv_smooth)
    m, k = q.shape
    n = w.weight.shape[0]
    if not x.is_cuda:
        y = (q.float() @ w.weight.float().t()) * sc[:, None] * w.row_scale.float()[None, :]
        if w.bias is not None:
            y = y + w.bias.float()
        if act == "gelu_tanh":
            y = R.gelu_tanh(y)
        elif act == "silu":
            y = torch.nn.functional.silu(y)
        if gate is not None:
            y = y * gate.float()
        if residual is not None:
            y = y + residual.float()
        y = y.to(torch.bfloat16)
        if out is not None:
            out.copy_(y)
            return out
        return y
    if out is None:
        out = torch.empty(m, n, dtype=torch.bfloat16, device=x.device)
    st = N.state(x.device)
    ws = st.gemm_workspace()
    rc = N.lib().b200_gemm(q.data_ptr(), w.weight.data_ptr(), out.data_ptr(), m, n, k, q.stride(0), w.weight.stride(0),
                           out.stride(0), 3, sc.data_ptr(), w.row_scale.data_ptr(), N.ptr(w.bias), N.ptr(gate), N.ptr(residual),
                           _ACT[act], 0, ws.data_ptr(), ws.numel(), st.status.data_ptr(), N.stream())
    N.check(rc, "b200_gemm")
    return out


# ---------------------------------------------------------------------------------------------
def quant_fp8_act(x: torch.Tensor, tile_rows: int = 128, mx: Optional[bool] = None) -> Fp8Act:
    """bf16 [M, K] -> e4m3 with one scale per 128 consecutive K values (fp32, or UE8M0 in the
    blocked layout with ``tile_rows`` rows per block when the UE8M0 mode is on)."""
    mx = fp8_mx() if mx is None else mx
    if not x.is_cuda:
        q, s = R.quant_fp8_act(x, pow2=mx)
        return Fp8Act(q, s)
    m, k = x.shape
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1
    q = torch.empty(m, k, dtype=torch.uint8, device=x.device)
    if mx:
        sf = _alloc_sf(m, k, tile_rows, x.device)
        N.check(N.lib().b200_quant_fp8(x.data_ptr(), q.data_ptr(), sf.data_ptr(), m, k, x.stride(0), tile_rows,
                                       N.stream()), "b200_quant_fp8")
        return Fp8Act(q, None, sf, tile_rows)
    s = torch.empty(m, k // 128, dtype=torch.float32, device=x.device)
    N.check(N.lib().b200_quant_fp8(x.data_ptr(), q.data_ptr(), s.data_ptr(), m, k, x.stride(0), 0, N.stream()),
            "b200_quant_fp8")
    return Fp8Act(q, s)


def quant_fp8_weight(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """bf16 [N, K] -> (e4m3 bytes, scales [ceil(N/128), K/128]) with one scale per 128x128 block."""
    if not w.is_cuda or fp8_mx():
        # UE8M0 mode: power-of-two scales; a load-time step, so plain tensor ops are fine
        return R.quant_fp8_weight(w, pow2=fp8_mx())
    n, k = w.shape
    w = w.to(torch.bfloat16).contiguous()
    q = torch.empty(n, k, dtype=torch.uint8, device=w.device)
    s = torch.empty((n + 127) // 128, k // 128, dtype=torch.float32, device=w.device)
    N.check(N.lib().b200_quant_fp8_weight(w.data_ptr(), q.data_ptr(), s.data_ptr(), n, k, N.stream()),
            "b200_quant_fp8_weight")
    return q, s


@dataclass
class SplitSum:
    """Result of a small-token GEMM whose K ranges were left unsummed in the GEMM scratch
    (``linear(..., defer=True)``): the consumer kernel (``glu``, ``rope_kv``) adds them while it
    reads, so no reduce kernel runs in between. Valid until the next GEMM on the device."""
    ws: torch.Tensor          # the device's GEMM scratch
    splits: int
    bn: int
    shape: tuple              # (tokens, features) of the product

    def part_args(self):
        return self.ws.data_ptr() + 16384, self.splits, self.bn


def _part_args(x):
    return x.part_args() if isinstance(x, SplitSum) else (None, 0, 0)


def _gemm_dtype(w: LinearWeight) -> int:
    return 2 if w.is_mx else 1 if w.is_fp8 else 0


def _scale_ptrs(x, w: LinearWeight):
    if not w.is_fp8:
        return None, None
    if w.is_mx:
        return x.sf.data_ptr(), w.sf.data_ptr()
    return x.scale.data_ptr(), w.scale.data_ptr()


def linear(x, w: LinearWeight, act: Optional[str] = None, gate: Optional[torch.Tensor] = None,
           residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
           splits: Optional[int] = None, defer: bool = False):
    """y = residual + gate * act(x @ W^T + bias), bf16 output [M, N].

    ``x`` is a bf16 tensor [M, K] or an :class:`Fp8Act`. With an fp8 weight a bf16 ``x`` is
    quantised on the fly (1x128 groups). ``gate`` is a per-output-feature vector [N].
    ``defer=True`` (device, plain product only): when the GEMM cuts all its tiles along K, return a
    :class:`SplitSum` for a consumer that adds the ranges itself instead of running the reduce kernel.
    """
    if isinstance(w, GgufWeight):
        if act is not None or gate is not None or residual is not None or isinstance(x, Fp8Act):
            raise ValueError("GGUF block weights take bf16 activations and no fused epilogue")
        return gguf_linear(x, w, out=out)
    if isinstance(w, Int8Weight):
        if isinstance(x, Fp8Act):
            raise ValueError("int8 weights take bf16 activations")
        return int8_linear(x, w, act, gate, residual, out)
    xd = x.data if isinstance(x, Fp8Act) else x
    if not xd.is_cuda:
        if isinstance(x, Fp8Act):
            y = R.linear(x.data, w.weight, w.scale, x.scale, w.bias, act, gate, residual)
        elif w.is_fp8:
            q, s = R.quant_fp8_act(x, pow2=fp8_mx())
            y = R.linear(q, w.weight, w.scale, s, w.bias, act, gate, residual)
        else:
            y = R.linear(x, w.host_f32(), None, None, w.bias, act, gate, residual)
        if out is not None:
            out.copy_(y)
            return out
        return y
    if w.is_fp8 and not isinstance(x, Fp8Act):
        x = quant_fp8_act(x, mx=w.is_mx)
        xd = x.data
    if not w.is_fp8 and isinstance(x, Fp8Act):
        raise ValueError("fp8 activations need an fp8 weight")
    if w.is_fp8 and (x.sf is not None) != w.is_mx:
        raise ValueError("activation and weight use different fp8 scale formats")
    m, k = xd.shape
    n = w.weight.shape[0]
    assert w.weight.shape[1] == k, (w.weight.shape, xd.shape)
    assert xd.stride(1) == 1 and w.weight.stride(1) == 1
    if out is None:
        out = torch.empty(m, n, dtype=torch.bfloat16, device=xd.device)
    fp8 = w.is_fp8
    L = N.lib()
    st = N.state(xd.device)
    ws = st.gemm_workspace()
    xs_ptr, ws_ptr = _scale_ptrs(x, w)
    if defer and m <= 128 and w.bias is None and act is None and gate is None and residual is None and splits is None:
        import ctypes as C
        info = (C.c_int * 4)()
        rc = L.b200_gemm_deferred(xd.data_ptr(), w.weight.data_ptr(), out.data_ptr(), m, n, k, xd.stride(0),
                                  w.weight.stride(0), out.stride(0), _gemm_dtype(w), xs_ptr, ws_ptr, ws.data_ptr(),
                                  ws.numel(), info, st.status.data_ptr(), N.stream())
        N.check(rc, "b200_gemm_deferred")
        return SplitSum(ws, int(info[1]), int(info[2]), (m, n)) if info[0] else out
    rc = L.b200_gemm(xd.data_ptr(), w.weight.data_ptr(), out.data_ptr(), m, n, k,
                     xd.stride(0), w.weight.stride(0), out.stride(0), _gemm_dtype(w),
                     xs_ptr, ws_ptr,
                     N.ptr(w.bias), N.ptr(gate), N.ptr(residual), _ACT[act], 0 if splits is None else splits,
                     ws.data_ptr(), ws.numel(), st.status.data_ptr(), N.stream())
    N.check(rc, "b200_gemm")
    return out


def norm(x: torch.Tensor, weight: Optional[torch.Tensor] = None, *, bias: Optional[torch.Tensor] = None,
         residual: Optional[torch.Tensor] = None, shift: Optional[torch.Tensor] = None,
         scale: Optional[torch.Tensor] = None, rows_per_batch: int = 0, eps: float = 1e-6,
         layernorm: bool = False, weight_plus_one: bool = False, emit_fp8: bool = False,
         emit_bf16: bool = True, fp8_tile_rows: int = 128):
    """(residual add +) RMSNorm / LayerNorm (+ affine) (+ AdaLN ``y * (1 + scale) + shift``).

    x [rows, dim] bf16. ``shift``/``scale`` are [batch, >= dim] with ``rows_per_batch`` rows
    sharing a batch entry. Returns ``(y, h, y_fp8)``: y bf16 (or None), h = x + residual (or
    None), y_fp8 an :class:`Fp8Act` (or None).
    """
    rows, dim = x.shape
    if not x.is_cuda:
        yf, h = R.norm(x, weight, bias, residual, shift, scale, rows_per_batch, eps, layernorm, weight_plus_one)
        y = yf.to(x.dtype)
        fq = None
        if emit_fp8:
            q, s = R.quant_fp8_act(y, pow2=fp8_mx())
            fq = Fp8Act(q, s)
        return (y if emit_bf16 else None), h, fq
    assert x.dtype == torch.bfloat16 and x.is_contiguous()
    y = torch.empty_like(x) if emit_bf16 else None
    h = torch.empty_like(x) if residual is not None else None
    q = s = None
    mx = emit_fp8 and fp8_mx()
    if emit_fp8:
        q = torch.empty(rows, dim, dtype=torch.uint8, device=x.device)
        s = _alloc_sf(rows, dim, fp8_tile_rows, x.device) if mx else \
            torch.empty(rows, dim // 128, dtype=torch.float32, device=x.device)
    mod_stride = 0
    if shift is not None or scale is not None:
        ref = shift if shift is not None else scale
        mod_stride = ref.stride(0) if ref.dim() > 1 else 0
    rc = N.lib().b200_norm(x.data_ptr(), N.ptr(residual), N.ptr(h), N.ptr(weight), N.ptr(bias),
                           N.ptr(shift), N.ptr(scale), N.ptr(y), N.ptr(q), N.ptr(s), rows, dim,
                           rows_per_batch, mod_stride, eps, int(layernorm), int(weight_plus_one),
                           fp8_tile_rows if mx else 0, N.stream())
    N.check(rc, "b200_norm")
    if not emit_fp8:
        return y, h, None
    return y, h, (Fp8Act(q, None, s, fp8_tile_rows) if mx else Fp8Act(q, s))


def glu(x: torch.Tensor, act: str = "silu", emit_fp8: bool = False, emit_bf16: bool = True,
        fp8_tile_rows: int = 128):
    """act(x[:, :F]) * x[:, F:] for x [rows, 2F]. Returns (y bf16 or None, y_fp8 or None)."""
    rows, f2 = x.shape
    f = f2 // 2
    if isinstance(x, SplitSum):
        dev = x.ws.device
        y = torch.empty(rows, f, dtype=torch.bfloat16, device=dev) if emit_bf16 else None
        q = s = None
        mx = emit_fp8 and fp8_mx()
        if emit_fp8:
            q = torch.empty(rows, f, dtype=torch.uint8, device=dev)
            s = _alloc_sf(rows, f, fp8_tile_rows, dev) if mx else torch.empty(rows, f // 128, dtype=torch.float32, device=dev)
        rc = N.lib().b200_glu(None, N.ptr(y), N.ptr(q), N.ptr(s), rows, f, 0 if act == "silu" else 1,
                              fp8_tile_rows if mx else 0, *x.part_args(), N.stream())
        N.check(rc, "b200_glu")
        if not emit_fp8:
            return y, None
        return y, (Fp8Act(q, None, s, fp8_tile_rows) if mx else Fp8Act(q, s))
    if not x.is_cuda:
        y = R.glu(x, act).to(x.dtype)
        fq = None
        if emit_fp8:
            q, s = R.quant_fp8_act(y, pow2=fp8_mx())
            fq = Fp8Act(q, s)
        return (y if emit_bf16 else None), fq
    assert x.is_contiguous() and x.dtype == torch.bfloat16
    y = torch.empty(rows, f, dtype=torch.bfloat16, device=x.device) if emit_bf16 else None
    q = s = None
    mx = emit_fp8 and fp8_mx()
    if emit_fp8:
        q = torch.empty(rows, f, dtype=torch.uint8, device=x.device)
        s = _alloc_sf(rows, f, fp8_tile_rows, x.device) if mx else \
            torch.empty(rows, f // 128, dtype=torch.float32, device=x.device)
    rc = N.lib().b200_glu(x.data_ptr(), N.ptr(y), N.ptr(q), N.ptr(s), rows, f, 0 if act == "silu" else 1,
                          fp8_tile_rows if mx else 0, None, 0, 0, N.stream())
    N.check(rc, "b200_glu")
    if not emit_fp8:
        return y, None
    return y, (Fp8Act(q, None, s, fp8_tile_rows) if mx else Fp8Act(q, s))


def rope_kv(qkv: torch.Tensor, positions: torch.Tensor, hq: int, hkv: int, d: int, *,
            k_cache: Optional[torch.Tensor] = None, v_cache: Optional[torch.Tensor] = None,
            slot_mapping: Optional[torch.Tensor] = None, rot: Optional[int] = None,
            theta: float = 10000.0, inv_freq: Optional[torch.Tensor] = None, style: int = 0,
            q_norm_w: Optional[torch.Tensor] = None, k_norm_w: Optional[torch.Tensor] = None,
            eps: float = 1e-6, want_kv: bool = False):
    """Optional QK RMSNorm + rotary embedding on a packed qkv activation [T, (hq + 2 hkv) d], and
    the K/V write into the page pool ([pages, hkv, page, d], slot = page_index * page + offset).
    Returns (q [T, hq, d], k [T, hkv, d] or None, v or None). ``qkv`` may be a :class:`SplitSum`."""
    part = qkv if isinstance(qkv, SplitSum) else None
    t = qkv.shape[0]
    rot = d if rot is None else rot
    if part is None and not qkv.is_cuda:
        x = qkv.float().reshape(t, hq + 2 * hkv, d)
        q, k, v = x[:, :hq], x[:, hq:hq + hkv], x[:, hq + hkv:]
        if q_norm_w is not None:
            q = q * torch.rsqrt((q * q).mean(-1, keepdim=True) + eps) * q_norm_w.float()
        if k_norm_w is not None:
            k = k * torch.rsqrt((k * k).mean(-1, keepdim=True) + eps) * k_norm_w.float()
        if rot > 0:
            fr = inv_freq if inv_freq is not None else R.rope_inv_freq(rot, theta, qkv.device)
            q = R.apply_rope(q, positions, fr, style)
            k = R.apply_rope(k, positions, fr, style)
        q, k, v = q.to(qkv.dtype), k.to(qkv.dtype), v.to(qkv.dtype)
        if k_cache is not None and slot_mapping is not None:
            page = k_cache.shape[2]
            ok = slot_mapping >= 0
            pg, off = (slot_mapping[ok] // page).long(), (slot_mapping[ok] % page).long()
            k_cache[pg, :, off] = k[ok]
            v_cache[pg, :, off] = v[ok]
        return q.contiguous(), (k.contiguous() if want_kv else None), (v.contiguous() if want_kv else None)
    dev = part.ws.device if part is not None else qkv.device
    assert part is not None or (qkv.is_contiguous() and qkv.dtype == torch.bfloat16)
    q = torch.empty(t, hq, d, dtype=torch.bfloat16, device=dev)
    k = torch.empty(t, hkv, d, dtype=torch.bfloat16, device=dev) if want_kv else None
    v = torch.empty(t, hkv, d, dtype=torch.bfloat16, device=dev) if want_kv else None
    page = k_cache.shape[2] if k_cache is not None else 16
    if slot_mapping is not None:
        assert slot_mapping.dtype == torch.int64
    assert positions.dtype == torch.int32
    rc = N.lib().b200_rope_kv(None if part is not None else qkv.data_ptr(), q.data_ptr(), N.ptr(k_cache), N.ptr(v_cache),
                              N.ptr(k), N.ptr(v), positions.data_ptr(), N.ptr(slot_mapping), N.ptr(q_norm_w),
                              N.ptr(k_norm_w), N.ptr(inv_freq), t, hq, hkv, d, rot, style, page, theta, eps,
                              *_part_args(qkv), N.stream())
    N.check(rc, "b200_rope_kv")
    return q, k, v


def attn_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                kv_lens: torch.Tensor, scale: Optional[float] = None, softcap: float = 0.0,
                window: int = 0, splits: Optional[int] = None, max_kv_len: Optional[int] = None,
                emit_fp8: bool = False, emit_bf16: bool = True):
    """One query token per sequence against a paged KV pool. q [B, hq, d] -> [B, hq, d].
    With ``emit_fp8`` the result is ``(out, Fp8Act of out.reshape(B, hq * d))``: quantised by the
    split-combine kernel itself when it runs (head dim 128, more than one KV split; ``out`` is then
    None unless ``emit_bf16``), by a separate kernel otherwise."""
    b, hq, d = q.shape
    hkv, page = k_cache.shape[1], k_cache.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    if not q.is_cuda:
        outs = []
        for i in range(b):
            ln = int(kv_lens[i])
            kk = R.gather_paged(k_cache, block_table[i], ln)
            vv = R.gather_paged(v_cache, block_table[i], ln)
            outs.append(R.attention(q[i:i + 1], kk, vv, causal=False, scale=scale, softcap=softcap,
                                    window=window))
        o = torch.cat(outs, 0).to(q.dtype)
        return (o, quant_fp8_act(o.reshape(b, hq * d))) if emit_fp8 else o
    assert block_table.dtype == torch.int32 and kv_lens.dtype == torch.int32
    L = N.lib()
    if splits is None:
        mk = max_kv_len if max_kv_len is not None else block_table.shape[1] * page
        splits = L.b200_attn_decode_pick_splits(b, hkv, mk)
    ws = None
    if splits > 1:
        ws = N.state(q.device).scratch(L.b200_attn_decode_workspace_bytes(b, hq, d, splits)).data_ptr()
    fused_q = emit_fp8 and d == 128 and splits > 1
    out = torch.empty_like(q) if (emit_bf16 or not fused_q) else None
    oq = osc = None
    mx = fp8_mx()
    if fused_q:
        oq = torch.empty(b, hq * d, dtype=torch.uint8, device=q.device)
        osc = _alloc_sf(b, hq * d, 128, q.device) if mx else torch.empty(b, hq, dtype=torch.float32, device=q.device)
    rc = L.b200_attn_decode(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), N.ptr(out),
                            block_table.data_ptr(), kv_lens.data_ptr(), b, hq, hkv, d, page,
                            block_table.shape[1], splits, ws, scale, softcap, window, N.ptr(oq), N.ptr(osc),
                            128 if (fused_q and mx) else 0, N.stream())
    N.check(rc, "b200_attn_decode", 2 if splits > 1 else 1)
    if not emit_fp8:
        return out
    if fused_q:
        return out, (Fp8Act(oq, None, osc, 128) if mx else Fp8Act(oq, osc))
    return out, quant_fp8_act(out.reshape(b, hq * d))


def attn_paged_biased(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                      kv_lens: torch.Tensor, cu_q: Optional[torch.Tensor], scale: Optional[float] = None,
                      softcap: float = 0.0, window: int = 0, alibi: Optional[torch.Tensor] = None,
                      sinks: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Paged causal attention with ALiBi slopes and / or per-head sink logits, which the attention
    kernels do not take: the sequences are gathered from the page pool and run through tensor ops
    on whichever device holds them. ``cu_q`` None means one query token per sequence (decode)."""
    nseq = kv_lens.numel()
    bounds = list(range(nseq + 1)) if cu_q is None else cu_q.tolist()
    lens = kv_lens.tolist()
    out = torch.empty_like(q)
    for i in range(nseq):
        a, b = bounds[i], bounds[i + 1]
        kk = R.gather_paged(k_cache, block_table[i], lens[i])
        vv = R.gather_paged(v_cache, block_table[i], lens[i])
        out[a:b] = R.attention(q[a:b], kk, vv, causal=True, scale=scale, softcap=softcap, window=window,
                               alibi=alibi, sinks=sinks).to(q.dtype)
    return out


def attn_prefill_paged(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                       block_table: torch.Tensor, kv_lens: torch.Tensor, cu_q: torch.Tensor,
                       max_q_len: int, causal: bool = True, scale: Optional[float] = None,
                       softcap: float = 0.0, window: int = 0) -> torch.Tensor:
    """Variable-length (chunked) prefill: q [total_q, hq, d] packed by cu_q; keys come from the page
    pool and include any cached prefix (kv_lens[i] >= q_len[i])."""
    tq, hq, d = q.shape
    hkv, page = k_cache.shape[1], k_cache.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    nseq = cu_q.numel() - 1
    if not q.is_cuda:
        out = torch.empty_like(q)
        for i in range(nseq):
            a, b = int(cu_q[i]), int(cu_q[i + 1])
            ln = int(kv_lens[i])
            kk = R.gather_paged(k_cache, block_table[i], ln)
            vv = R.gather_paged(v_cache, block_table[i], ln)
            out[a:b] = R.attention(q[a:b], kk, vv, causal=causal, scale=scale, softcap=softcap,
                                   window=window).to(q.dtype)
        return out
    out = torch.empty_like(q)
    rc = N.lib().b200_attn_prefill(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
                                   block_table.data_ptr(), kv_lens.data_ptr(), cu_q.data_ptr(), None,
                                   nseq, max_q_len, 0, 0, hq, hkv, d, page, block_table.shape[1], 1,
                                   int(causal), window, scale, softcap, N.stream())
    N.check(rc, "b200_attn_prefill")
    return out


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = False,
              scale: Optional[float] = None, softcap: float = 0.0, window: int = 0,
              int8: Optional[bool] = None) -> torch.Tensor:
    """Dense attention for one sequence: q [Tq, hq, d], k/v [Tk, hkv, d] -> [Tq, hq, d].
    ``int8`` (default: flag ``sage_attention``) selects the int8 Q K^T mode of the tcgen05 kernel."""
    tq, hq, d = q.shape
    tk, hkv, _ = k.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    if not q.is_cuda:
        return R.attention(q, k, v, causal, scale, softcap, window).to(q.dtype)
    assert q.is_contiguous() and k.is_contiguous() and v.is_contiguous()
    out = torch.empty_like(q)
    dense_tc = d == 128 and hq == hkv and not causal and softcap == 0.0 and window <= 0 and tk >= 256 and _tc_attention()
    from .. import config
    if dense_tc and config.get("fa_attention"):
        # long bidirectional sequences (DiT blocks): two query tiles per CTA, S / P / O in TMEM
        L = N.lib()
        i8 = int(config.get("sage_attention") if int8 is None else int8)
        ws = N.state(q.device).scratch(L.b200_attn_fa_workspace_bytes(1, hq, tq, tk, i8))
        rc = L.b200_attn_fa(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), 1, tq, tk, hq, float(scale), i8,
                            ws.data_ptr(), N.state(q.device).status.data_ptr(), N.stream())
        N.check(rc, "b200_attn_fa", 5 if i8 else 2)
        return out
    if dense_tc:
        # long bidirectional sequences (DiT blocks): tcgen05 kernel, V consumed transposed
        L = N.lib()
        vt = torch.empty(L.b200_attn_tc_workspace_bytes(1, hq, tk), dtype=torch.uint8, device=q.device)
        rc = L.b200_attn_tc(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), 1, tq, tk, hq, float(scale),
                            vt.data_ptr(), N.state(q.device).status.data_ptr(), N.stream())
        N.check(rc, "b200_attn_tc")
        return out
    rc = N.lib().b200_attn_prefill(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), None, None,
                                   None, None, 1, tq, tq, tk, hq, hkv, d, 16, 0, 0, int(causal), window,
                                   scale, softcap, N.stream())
    N.check(rc, "b200_attn_prefill")
    return out


def embedding(ids: torch.Tensor, table: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    if not table.is_cuda:
        y = table[ids.long()]
        return y if scale == 1.0 else (y.float() * scale).to(table.dtype)
    assert ids.dtype == torch.int32 and table.dtype == torch.bfloat16
    t = ids.numel()
    out = torch.empty(t, table.shape[1], dtype=torch.bfloat16, device=table.device)
    N.check(N.lib().b200_embedding(ids.data_ptr(), table.data_ptr(), out.data_ptr(), t, table.shape[1],
                                   table.shape[0], scale, N.stream()), "b200_embedding")
    return out


def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Row-wise argmax of [rows, vocab] (bf16 or fp32) -> int32 [rows]; ties resolve to the lowest id."""
    if not logits.is_cuda:
        r = logits.float().argmax(dim=-1).to(torch.int32)
        if out is not None:
            out.copy_(r)
            return out
        return r
    rows, vocab = logits.shape
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    N.check(N.lib().b200_argmax(logits.data_ptr(), out.data_ptr(), rows, vocab, logits.stride(0),
                                1 if logits.dtype == torch.float32 else 0, N.stream()), "b200_argmax")
    return out


def sample_tokens(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
                  min_p: torch.Tensor, seed: torch.Tensor, counter: torch.Tensor) -> torch.Tensor:
    """One token per row of ``logits`` [rows, vocab] (fp32 or bf16): temperature -> top-k -> top-p ->
    min-p -> draw, all on the device. Per-row parameters: ``temperature`` fp32 (<= 0: argmax),
    ``top_k`` int32 (<= 0: off), ``top_p`` / ``min_p`` fp32 (<= 0: off), ``seed`` / ``counter`` int64
    (the draw is a pure function of the two, so a request's stream is reproducible). int32 [rows]."""
    rows, vocab = logits.shape
    if not logits.is_cuda:
        out = torch.empty(rows, dtype=torch.int32)
        for r in range(rows):
            t = float(temperature[r])
            if t <= 0:
                out[r] = int(logits[r].float().argmax())
                continue
            keep = R.sampling_keep_mask(logits[r], t, int(top_k[r]), float(top_p[r]), float(min_p[r]))
            lg = (logits[r].float() / max(t, 1e-6)).masked_fill(~keep, float("-inf"))
            g = torch.Generator().manual_seed((int(seed[r]) * 1000003 + int(counter[r])) % (2 ** 63))
            out[r] = int(torch.multinomial(torch.softmax(lg, -1), 1, generator=g)[0])
        return out
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    assert logits.stride(1) == 1 and logits.dtype in (torch.float32, torch.bfloat16)
    N.check(N.lib().b200_sample(logits.data_ptr(), 1 if logits.dtype == torch.float32 else 0, logits.stride(0), rows, vocab,
                                temperature.data_ptr(), top_k.data_ptr(), top_p.data_ptr(), min_p.data_ptr(),
                                seed.data_ptr(), counter.data_ptr(), out.data_ptr(), N.stream()), "b200_sample")
    return out


def repetition_penalty_(logits: torch.Tensor, history: torch.Tensor, hist_len: torch.Tensor,
                        penalty: torch.Tensor) -> torch.Tensor:
    """In place: logits[b, t] /= p if > 0 else *= p for every token id t in history[b, :hist_len[b]]."""
    rows, vocab = logits.shape
    if not logits.is_cuda:
        for b in range(rows):
            p = float(penalty[b])
            if p == 1.0:
                continue
            ids = torch.unique(history[b, : int(hist_len[b])].long())
            ids = ids[(ids >= 0) & (ids < vocab)]
            vals = logits[b, ids]
            logits[b, ids] = torch.where(vals > 0, vals / p, vals * p)
        return logits
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    N.check(N.lib().b200_repetition_penalty(logits.data_ptr(), history.data_ptr(), hist_len.data_ptr(),
                                            history.shape[1], rows, vocab, penalty.data_ptr(), N.stream()),
            "b200_repetition_penalty")
    return logits


def cfg_euler_step(z: torch.Tensor, cond: torch.Tensor, uncond: Optional[torch.Tensor], guidance: float,
                   dt: float) -> torch.Tensor:
    """In place on fp32 latents: z += (g * cond + (1 - g) * uncond) * dt (uncond None -> v = cond)."""
    if not z.is_cuda:
        z.copy_(R.cfg_euler(z, cond, uncond, guidance, dt))
        return z
    assert z.dtype == torch.float32 and cond.dtype == torch.bfloat16
    N.check(N.lib().b200_cfg_euler(z.data_ptr(), cond.data_ptr(), N.ptr(uncond), z.numel(), guidance, dt,
                                   N.stream()), "b200_cfg_euler")
    return z


_RENORM_SCRATCH: dict = {}


def cfg_renorm_euler_step(z: torch.Tensor, cond: torch.Tensor, uncond: torch.Tensor, guidance: float, dt: float,
                          renorm_min: float = 0.0) -> torch.Tensor:
    """In place on fp32 latents: guided = uncond + g (cond - uncond), rescaled by ONE factor
    clamp(||cond|| / ||guided||, renorm_min, 1) for the whole tensor, then z += guided dt. cond / uncond
    bf16 or fp32. Two launches on the device (norms + scale, then the update)."""
    if not z.is_cuda:
        z.copy_(R.cfg_renorm_euler(z, cond, uncond, guidance, dt, renorm_min))
        return z
    assert z.dtype == torch.float32 and z.is_contiguous() and cond.dtype == uncond.dtype and cond.dtype in (torch.bfloat16, torch.float32)
    assert cond.is_contiguous() and uncond.is_contiguous() and cond.numel() == z.numel() == uncond.numel()
    key = (z.device.index, N.stream())
    scratch = _RENORM_SCRATCH.get(key)
    if scratch is None:
        nbytes = int(N.bind("b200_cfg_renorm_scratch_bytes", C.c_longlong, [])())
        scratch = torch.zeros((nbytes + 7) // 8, dtype=torch.int64, device=z.device)
        _RENORM_SCRATCH[key] = scratch
    fn = N.bind("b200_cfg_renorm_euler", C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_longlong, C.c_float, C.c_float,
                                                   C.c_float, C.c_void_p, C.c_void_p])
    N.check(fn(z.data_ptr(), cond.data_ptr(), uncond.data_ptr(), int(cond.dtype == torch.bfloat16), z.numel(), guidance, dt,
               renorm_min, scratch.data_ptr(), N.stream()), "b200_cfg_renorm_euler")
    return z


def cfg_rownorm_euler_step(z: torch.Tensor, cond: torch.Tensor, uncond: torch.Tensor, guidance: float, dt: float,
                           eps: float = 1e-12) -> torch.Tensor:
    """In place on fp32 latents [..., D]: guided rows rescaled to the norm of the conditional rows
    (ratio per row of the last dimension), then z += guided dt. One launch on the device."""
    if not z.is_cuda:
        z.copy_(R.cfg_rownorm_euler(z, cond, uncond, guidance, dt, eps))
        return z
    assert z.dtype == torch.float32 and z.is_contiguous() and cond.dtype == uncond.dtype and cond.dtype in (torch.bfloat16, torch.float32)
    assert cond.is_contiguous() and uncond.is_contiguous() and cond.shape == z.shape == uncond.shape
    d = z.shape[-1]
    fn = N.bind("b200_cfg_rownorm_euler", C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_longlong, C.c_int, C.c_float,
                                                    C.c_float, C.c_float, C.c_void_p])
    N.check(fn(z.data_ptr(), cond.data_ptr(), uncond.data_ptr(), int(cond.dtype == torch.bfloat16), z.numel() // d, d, guidance, dt,
               eps, N.stream()), "b200_cfg_rownorm_euler")
    return z


def lincomb(terms: list, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """sum_i coef_i * x_i for ``terms`` = [(coef, fp32 tensor), ...] (at most eight, same shape): the update
    of a multistep solver in one pass over the latents. ``out`` may be one of the operands."""
    xs = [t for _, t in terms]
    if out is None:
        out = torch.empty_like(xs[0])
    if not xs[0].is_cuda or len(xs) > 8 or any(t.dtype != torch.float32 or not t.is_contiguous() or t.data_ptr() % 16 for t in xs + [out]):
        acc = sum(float(c) * t.float() for c, t in terms)
        out.copy_(acc.to(out.dtype))
        return out
    ptrs = (C.c_void_p * 8)(*[t.data_ptr() for t in xs])
    coefs = (C.c_float * 8)(*[float(c) for c, _ in terms])
    fn = N.bind("b200_lincomb", C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_longlong, C.c_void_p])
    N.check(fn(out.data_ptr(), ptrs, coefs, len(xs), out.numel(), N.stream()), "b200_lincomb")
    return out


def gated_residual(x: torch.Tensor, y: torch.Tensor, gate: torch.Tensor, rows_per_batch: int = 0) -> torch.Tensor:
    """x + gate[batch] * y for [rows, dim] bf16 with gate [batch, >= dim]."""
    rows, dim = x.shape
    if not x.is_cuda:
        rpb = rows_per_batch if rows_per_batch > 0 else rows
        idx = torch.arange(rows) // rpb
        g = gate.float().reshape(-1, gate.shape[-1])[idx][:, :dim]
        return (x.float() + g * y.float()).to(x.dtype)
    out = torch.empty_like(x)
    ms = gate.stride(0) if gate.dim() > 1 else 0
    N.check(N.lib().b200_gated_residual(x.data_ptr(), y.data_ptr(), gate.data_ptr(), out.data_ptr(), rows,
                                        dim, rows_per_batch, ms, N.stream()), "b200_gated_residual")
    return out


def fill_random_(t: torch.Tensor, seed: int, std: float = 0.02) -> torch.Tensor:
    """Deterministic synthetic fill: bf16 ~ N(0, std); uint8 tensors get e4m3 bytes of unit-variance
    values scaled by 112 (so a block scale of std / 112 reproduces N(0, std))."""
    if not t.is_cuda:
        g = torch.Generator().manual_seed(seed)
        if t.dtype == torch.uint8:
            v = (torch.randn(t.shape, generator=g) * 112.0).clamp(-448, 448).to(torch.float8_e4m3fn)
            t.copy_(v.view(torch.uint8))
        else:
            t.copy_((torch.randn(t.shape, generator=g) * std).to(t.dtype))
        return t
    assert t.is_contiguous()
    N.check(N.lib().b200_fill_random(t.data_ptr(), t.numel(), seed, std, 1 if t.dtype == torch.uint8 else 0,
                                     N.stream()), "b200_fill_random")
    return t


def dit_qkv(qkv: torch.Tensor, hq: int, hkv: int, d: int, *, q_norm_w: Optional[torch.Tensor] = None,
            k_norm_w: Optional[torch.Tensor] = None, cos: Optional[torch.Tensor] = None,
            sin: Optional[torch.Tensor] = None, eps: float = 1e-6):
    """Split packed qkv [T, (hq + 2 hkv) d] into q [T, hq, d], k, v [T, hkv, d] with optional per-head
    RMSNorm on q / k and interleaved-pair rotary embedding from per-token tables cos / sin [T, d/2]."""
    t = qkv.shape[0]
    if not qkv.is_cuda:
        x = qkv.float().reshape(t, hq + 2 * hkv, d)
        q, k, v = x[:, :hq], x[:, hq:hq + hkv], x[:, hq + hkv:]
        if q_norm_w is not None:
            q = q * torch.rsqrt((q * q).mean(-1, keepdim=True) + eps) * q_norm_w.float()
        if k_norm_w is not None:
            k = k * torch.rsqrt((k * k).mean(-1, keepdim=True) + eps) * k_norm_w.float()
        if cos is not None:
            def rot(z):
                a, b = z[..., 0::2], z[..., 1::2]
                c, s = cos.float()[:, None, :], sin.float()[:, None, :]
                return torch.stack([a * c - b * s, b * c + a * s], dim=-1).flatten(-2)
            q, k = rot(q), rot(k)
        return q.to(qkv.dtype).contiguous(), k.to(qkv.dtype).contiguous(), v.to(qkv.dtype).contiguous()
    assert qkv.dtype == torch.bfloat16 and qkv.stride(1) == 1
    q = torch.empty(t, hq, d, dtype=torch.bfloat16, device=qkv.device)
    k = torch.empty(t, hkv, d, dtype=torch.bfloat16, device=qkv.device)
    v = torch.empty(t, hkv, d, dtype=torch.bfloat16, device=qkv.device)
    if cos is not None:
        assert cos.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous()
    N.check(N.lib().b200_dit_qkv(qkv.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), N.ptr(q_norm_w),
                                 N.ptr(k_norm_w), N.ptr(cos), N.ptr(sin), t, hq, hkv, d, qkv.stride(0), eps,
                                 N.stream()), "b200_dit_qkv")
    return q, k, v


# ---------------------------------------------------------------------------------------------
# mixture of experts
# ---------------------------------------------------------------------------------------------
def moe_route(logits: torch.Tensor, bias: Optional[torch.Tensor], top_k: int, *, n_group: int = 1,
              topk_group: int = 1, sigmoid: bool = False, norm_topk: bool = False,
              scale: float = 1.0) -> tuple[torch.Tensor, torch.Tensor]:
    """Router: logits [T, E] (fp32 or bf16) -> (expert ids int32 [T, k], weights fp32 [T, k]),
    entirely on the device (see :func:`reference.moe_route` for the exact rule)."""
    if not logits.is_cuda:
        return R.moe_route(logits, bias, top_k, n_group, topk_group, sigmoid, norm_topk, scale)
    t, e = logits.shape
    assert logits.is_contiguous() and logits.dtype in (torch.float32, torch.bfloat16)
    ids = torch.empty(t, top_k, dtype=torch.int32, device=logits.device)
    w = torch.empty(t, top_k, dtype=torch.float32, device=logits.device)
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.is_contiguous()
    rc = N.lib().b200_moe_route(logits.data_ptr(), 1 if logits.dtype == torch.bfloat16 else 0, N.ptr(bias),
                                ids.data_ptr(), w.data_ptr(), t, e, top_k, n_group, topk_group,
                                1 if sigmoid else 0, 1 if norm_topk else 0, float(scale), N.stream())
    N.check(rc, "b200_moe_route")
    return ids, w


def moe_capacity(tokens: int) -> int:
    """Slots per expert for a chunk of ``tokens`` (a token picks an expert at most once)."""
    for c in (16, 32, 64, 128):
        if tokens <= c:
            return c
    raise ValueError("MoE chunks hold at most 128 tokens")


def moe_dispatch(x: torch.Tensor, topk_ids: torch.Tensor, e0: int, e_local: int, capacity: int,
                 xs: torch.Tensor, slot_of: Optional[torch.Tensor] = None,
                 counts: Optional[torch.Tensor] = None, chunks: int = 1) -> tuple[torch.Tensor, torch.Tensor]:
    """Copy each token row into a slot of every local expert that it selected.

    Tokens are taken in ``chunks`` runs of at most 128; expert e owns block ``e * chunks + c`` of
    ``capacity`` slots for run c. ``xs`` [e_local * chunks * capacity, dim] is a caller-owned buffer
    (slots without a token keep stale, finite values). Returns (slot_of int32 [T, k] with -1 for
    remote experts, counts int32 [e_local * chunks])."""
    t, k = topk_ids.shape
    dim = x.shape[1]
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous()
    assert xs.shape == (e_local * chunks * capacity, dim)
    chunk_tokens = 128 if chunks > 1 else max(t, 1)
    if slot_of is None:
        slot_of = torch.empty(t, k, dtype=torch.int32, device=x.device)
    if counts is None:
        counts = torch.empty(e_local * chunks, dtype=torch.int32, device=x.device)
    rc = N.lib().b200_moe_dispatch(x.data_ptr(), xs.data_ptr(), topk_ids.data_ptr(), slot_of.data_ptr(),
                                   counts.data_ptr(), t, k, dim, e0, e_local, capacity, chunks, chunk_tokens,
                                   N.stream())
    N.check(rc, "b200_moe_dispatch")
    return slot_of, counts


def grouped_linear(x, w: LinearWeight, groups: int, act: Optional[str] = None,
                   counts: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                   chunks: int = 1) -> torch.Tensor:
    """Per-group y[b] = x[b] @ w[b // chunks]^T in one launch. ``x`` [groups * chunks * m, K] (bf16
    or Fp8Act, m in {16, 32, 64, 128}), ``w`` stacked [groups * N, K]; token blocks with
    ``counts[b] == 0`` are skipped."""
    xd = x.data if isinstance(x, Fp8Act) else x
    m = xd.shape[0] // (groups * chunks)
    k = xd.shape[1]
    n = w.weight.shape[0] // groups
    if not xd.is_cuda:
        ys = []
        for b in range(groups * chunks):
            g = b // chunks
            wg = w.weight[g * n:(g + 1) * n]
            if w.is_fp8:
                sg = w.scale[g * (n // 128):(g + 1) * (n // 128)]
                if isinstance(x, Fp8Act):
                    q, s = x.data[b * m:(b + 1) * m], x.scale[b * m:(b + 1) * m]
                else:
                    q, s = R.quant_fp8_act(xd[b * m:(b + 1) * m], pow2=fp8_mx())
                ys.append(R.linear(q, wg, sg, s, None, act, None, None))
            else:
                ys.append(R.linear(xd[b * m:(b + 1) * m], wg, None, None, None, act, None, None))
        return torch.cat(ys)
    if w.is_fp8 and not isinstance(x, Fp8Act):
        x = quant_fp8_act(x, tile_rows=m, mx=w.is_mx)
        xd = x.data
    if w.is_mx and x.tile_rows != m:
        raise ValueError("UE8M0 activations of a grouped GEMM need one scale-factor block per group")
    assert xd.is_contiguous() and w.weight.is_contiguous() and w.weight.shape[1] == k
    if out is None:
        out = torch.empty(groups * chunks * m, n, dtype=torch.bfloat16, device=xd.device)
    fp8 = w.is_fp8
    st = N.state(xd.device)
    ws = st.gemm_workspace()
    xs_ptr, ws_ptr = _scale_ptrs(x, w)
    rc = N.lib().b200_gemm_grouped(xd.data_ptr(), w.weight.data_ptr(), out.data_ptr(), groups, m, n, k,
                                   _gemm_dtype(w), xs_ptr, ws_ptr, _ACT[act], N.ptr(counts), chunks,
                                   ws.data_ptr(), ws.numel(), st.status.data_ptr(), N.stream())
    N.check(rc, "b200_gemm_grouped")
    return out


@dataclass
class MoePlan:
    """Device-side result of :func:`moe_dispatch_dynamic`."""
    slot_of: torch.Tensor        # int32 [T, k], -1 for remote experts
    block_group: torch.Tensor    # int32 [max_blocks]: local expert of every block
    dyn_blocks: torch.Tensor     # int32 [1]: blocks in use
    cap: int
    max_blocks: int


def moe_block_capacity(tokens: int, top_k: int, num_experts: int) -> int:
    """Slots per block: about twice the expected tokens per expert, a power of two in [16, 128]."""
    want = max(1, 2 * tokens * top_k // max(num_experts, 1))
    for c in (16, 32, 64, 128):
        if want <= c:
            return c
    return 128


def moe_dispatch_dynamic(x: torch.Tensor, topk_ids: torch.Tensor, e0: int, e_local: int, cap: int,
                         xs: torch.Tensor) -> MoePlan:
    """Variable-size dispatch: every local expert gets as many ``cap``-slot blocks as its tokens
    need, packed back to back in ``xs`` [max_blocks * cap, dim] (``max_blocks`` =
    ceil(T k / cap) + e_local covers every routing). No host round trip."""
    t, k = topk_ids.shape
    dim = x.shape[1]
    max_blocks = xs.shape[0] // cap
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous()
    assert max_blocks >= (t * k + cap - 1) // cap + e_local
    dev = x.device
    slot_of = torch.empty(t, k, dtype=torch.int32, device=dev)
    scratch = torch.empty(2 * e_local + t * k, dtype=torch.int32, device=dev)
    block_group = torch.zeros(max_blocks, dtype=torch.int32, device=dev)
    dyn = torch.empty(1, dtype=torch.int32, device=dev)
    rc = N.lib().b200_moe_dispatch_dynamic(x.data_ptr(), xs.data_ptr(), topk_ids.data_ptr(), slot_of.data_ptr(),
                                           scratch.data_ptr(), block_group.data_ptr(), dyn.data_ptr(), t, k, dim, e0,
                                           e_local, cap, max_blocks, N.stream())
    N.check(rc, "b200_moe_dispatch_dynamic")
    return MoePlan(slot_of, block_group, dyn, cap, max_blocks)


def grouped_linear_dynamic(x, w: LinearWeight, groups: int, plan: MoePlan, act: Optional[str] = None) -> torch.Tensor:
    """Grouped GEMM over the blocks of a :class:`MoePlan`: block b of ``x`` [max_blocks * cap, K]
    times the weights of expert ``plan.block_group[b]``; only the blocks in use are computed."""
    if w.is_fp8 and not isinstance(x, Fp8Act):
        x = quant_fp8_act(x, tile_rows=plan.cap, mx=w.is_mx)
    xd = x.data if isinstance(x, Fp8Act) else x
    if w.is_mx and x.tile_rows != plan.cap:
        raise ValueError("UE8M0 activations of a grouped GEMM need one scale-factor block per token block")
    k = xd.shape[1]
    n = w.weight.shape[0] // groups
    assert xd.is_cuda and xd.is_contiguous() and xd.shape[0] == plan.max_blocks * plan.cap and w.weight.shape[1] == k
    out = torch.empty(plan.max_blocks * plan.cap, n, dtype=torch.bfloat16, device=xd.device)
    xs_ptr, ws_ptr = _scale_ptrs(x, w)
    rc = N.lib().b200_gemm_grouped_dynamic(xd.data_ptr(), w.weight.data_ptr(), out.data_ptr(), groups, plan.max_blocks,
                                           plan.cap, n, k, _gemm_dtype(w), xs_ptr, ws_ptr, _ACT[act],
                                           plan.block_group.data_ptr(), plan.dyn_blocks.data_ptr(),
                                           N.state(xd.device).status.data_ptr(), N.stream())
    N.check(rc, "b200_gemm_grouped_dynamic")
    return out


def moe_combine(y: torch.Tensor, slot_of: torch.Tensor, topk_w: torch.Tensor, out: torch.Tensor,
                accumulate: bool = False) -> torch.Tensor:
    """out[t] (+)= sum_k topk_w[t, k] * y[slot_of[t, k]] over the locally computed slots."""
    t, k = slot_of.shape
    dim = y.shape[1]
    assert y.is_cuda and y.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and out.is_contiguous()
    rc = N.lib().b200_moe_combine(y.data_ptr(), slot_of.data_ptr(), topk_w.data_ptr(), out.data_ptr(), t, k, dim,
                                  1 if accumulate else 0, N.stream())
    N.check(rc, "b200_moe_combine")
    return out


# ---------------------------------------------------------------------------------------------
# multi-head latent attention
# ---------------------------------------------------------------------------------------------
MLA_LATENT = 512
MLA_ROPE = 64
MLA_ROW = MLA_LATENT + MLA_ROPE


def colbatched_linear(x: torch.Tensor, w: torch.Tensor, groups: int, x_koff: int, out: torch.Tensor,
                      out_stride: int) -> torch.Tensor:
    """Per-group projection of one token block without a head-major transpose:
    ``out[t, g * out_stride + j] = sum_i x[t, g * x_koff + i] * w[g * n + j, i]`` with ``w`` stacked
    [groups * n, k] bf16, at most 128 tokens per call (longer inputs are processed in blocks)."""
    t = x.shape[0]
    n, k = w.shape[0] // groups, w.shape[1]
    if not x.is_cuda:
        xf, wf = x.float(), w.float()
        for g in range(groups):
            out[:, g * out_stride:g * out_stride + n] = (xf[:, g * x_koff:g * x_koff + k] @ wf[g * n:(g + 1) * n].t()).to(out.dtype)
        return out
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.stride(1) == 1 and out.stride(1) == 1
    st = N.state(x.device)
    ws = st.gemm_workspace()
    for t0 in range(0, t, 128):
        m = min(128, t - t0)
        xb, ob = x[t0:t0 + m], out[t0:t0 + m]
        rc = N.lib().b200_gemm_colbatched(xb.data_ptr(), w.data_ptr(), ob.data_ptr(), groups, m, n, k, x.stride(0),
                                          x_koff, out.stride(0), out_stride, ws.data_ptr(), ws.numel(),
                                          st.status.data_ptr(), N.stream())
        N.check(rc, "b200_gemm_colbatched")
    return out


def msda(value: torch.Tensor, shapes: list, offsets: torch.Tensor, logits: torch.Tensor, ref: torch.Tensor) -> torch.Tensor:
    """Multi-scale deformable attention between its linear layers: softmax over the sampling points,
    sampling locations from the reference boxes / points, bilinear gathers and the weighted sum, one
    kernel on the device (csrc/kernels/msda.cu); see :func:`reference.msda` for the shapes. Returns
    [B, Q, heads * D] in the dtype of ``value``."""
    if not value.is_cuda:
        return R.msda(value, shapes, offsets, logits, ref).to(value.dtype)
    b, rows, heads, d = value.shape
    _, q, _, lv, pts, _ = offsets.shape
    assert value.dtype in (torch.bfloat16, torch.float32) and sum(h * w for h, w in shapes) == rows and len(shapes) == lv
    value = value.contiguous()
    offsets, logits, ref = offsets.float().contiguous(), logits.float().contiguous(), ref.float().contiguous()
    sh = torch.tensor([[h, w] for h, w in shapes], dtype=torch.int32)
    st = torch.cumsum(torch.tensor([0] + [h * w for h, w in shapes[:-1]], dtype=torch.int32), 0).to(torch.int32)
    meta = torch.cat([sh.reshape(-1), st]).to(value.device)
    out = torch.empty(b, q, heads * d, dtype=value.dtype, device=value.device)
    fn = N.bind("b200_msda", C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p,
                                       C.c_void_p, C.c_void_p] + [C.c_int] * 7 + [C.c_void_p])
    rc = fn(value.data_ptr(), int(value.dtype == torch.bfloat16), offsets.data_ptr(), logits.data_ptr(), ref.data_ptr(),
            ref.shape[-1], int(ref.dim() == 4), meta.data_ptr(), meta.data_ptr() + 8 * lv, out.data_ptr(), b, rows, q, heads, d, lv,
            pts, N.stream())
    N.check(rc, "b200_msda")
    return out


def mla_prep(kv: torch.Tensor, kv_norm_w: torch.Tensor, q: torch.Tensor, q_abs: torch.Tensor,
             cache: Optional[torch.Tensor], positions: torch.Tensor, slot_mapping: Optional[torch.Tensor],
             inv_freq: torch.Tensor, heads: int, q_stride: int, q_rope_off: int, eps: float = 1e-6,
             rope_mscale: float = 1.0) -> None:
    """Latent RMSNorm + RoPE of the shared key part + cache write ([pages, page, 576] flattened to
    slots), and RoPE of each head's q_pe into ``q_abs[:, :, 512:]``. Interleaved-pair rotation."""
    t = kv.shape[0]
    if not kv.is_cuda:
        c = kv[:, :MLA_LATENT].float()
        c = c * torch.rsqrt((c * c).mean(-1, keepdim=True) + eps) * kv_norm_w.float()
        kpe = R.apply_rope(kv[:, MLA_LATENT:].float().unsqueeze(1), positions, inv_freq, 1)[:, 0] * 1.0
        qpe = q.reshape(t, heads, q_stride)[:, :, q_rope_off:q_rope_off + MLA_ROPE].float()
        qpe = R.apply_rope(qpe, positions, inv_freq, 1)
        if rope_mscale != 1.0:
            kpe, qpe = kpe * rope_mscale, qpe * rope_mscale
        q_abs[:, :, MLA_LATENT:] = qpe.to(q_abs.dtype)
        if cache is not None and slot_mapping is not None:
            ok = slot_mapping >= 0
            flat = cache.view(-1, MLA_ROW)
            flat[slot_mapping[ok].long()] = torch.cat([c, kpe], dim=-1).to(cache.dtype)[ok]
        return
    assert kv.is_contiguous() and q.is_contiguous() and q_abs.is_contiguous() and positions.dtype == torch.int32
    assert inv_freq.dtype == torch.float32 and inv_freq.numel() == MLA_ROPE // 2
    if slot_mapping is not None:
        assert slot_mapping.dtype == torch.int64
    rc = N.lib().b200_mla_prep(kv.data_ptr(), kv_norm_w.data_ptr(), q.data_ptr(), q_abs.data_ptr(), N.ptr(cache),
                               positions.data_ptr(), N.ptr(slot_mapping), inv_freq.data_ptr(), t, heads, q_stride,
                               q_rope_off, eps, rope_mscale, N.stream())
    N.check(rc, "b200_mla_prep")


def mla_attn(q_abs: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, kv_lens: torch.Tensor,
             scale: float, row_seq: Optional[torch.Tensor] = None, max_kv_len: Optional[int] = None,
             splits: Optional[int] = None) -> torch.Tensor:
    """Multi-query attention of absorbed queries [rows, heads, 576] over the latent cache
    [pages, page, 576]; row r attends to the first ``kv_lens[r]`` tokens of block-table row
    ``row_seq[r]`` (identity when None). Returns the latent outputs [rows, heads, 512]."""
    rows, heads, _ = q_abs.shape
    page = cache.shape[1]
    if not q_abs.is_cuda:
        out = torch.zeros(rows, heads, MLA_LATENT, dtype=q_abs.dtype)
        for r in range(rows):
            n = int(kv_lens[r])
            if n == 0:
                continue
            sq = int(row_seq[r]) if row_seq is not None else r
            npg = (n + page - 1) // page
            lat = cache[block_table[sq, :npg].long()].reshape(-1, MLA_ROW)[:n].float()
            sc = (q_abs[r].float() @ lat.t()) * scale
            out[r] = (torch.softmax(sc, dim=-1) @ lat[:, :MLA_LATENT]).to(out.dtype)
        return out
    assert q_abs.is_contiguous() and cache.is_contiguous() and block_table.dtype == torch.int32
    assert kv_lens.dtype == torch.int32 and (row_seq is None or row_seq.dtype == torch.int32)
    L = N.lib()
    if splits is None:
        mk = max_kv_len if max_kv_len else block_table.shape[1] * page
        splits = L.b200_mla_pick_splits(rows, heads, int(mk))
    out = torch.empty(rows, heads, MLA_LATENT, dtype=torch.bfloat16, device=q_abs.device)
    ws = None
    if splits > 1:
        ws = torch.empty(L.b200_mla_workspace_bytes(rows, heads, splits), dtype=torch.uint8, device=q_abs.device)
    rc = L.b200_mla_attn(q_abs.data_ptr(), cache.data_ptr(), out.data_ptr(), block_table.data_ptr(),
                         kv_lens.data_ptr(), N.ptr(row_seq), rows, heads, page, block_table.stride(0), splits,
                         N.ptr(ws), float(scale), N.stream())
    N.check(rc, "b200_mla_attn")
    return out


# ---------------------------------------------------------------------------------------------
# GGUF block-quantised weights kept in their file layout on the device
# ---------------------------------------------------------------------------------------------
GGML_Q8_0, GGML_Q4_K = 8, 12
_GGUF_ROW = {GGML_Q8_0: (32, 34), GGML_Q4_K: (256, 144)}      # type -> (values per block, bytes per block)
GGUF_GEMV_MAX_TOKENS = 16


@dataclass
class GgufWeight:
    """A [N, K] weight as raw ggml blocks: ``blocks`` uint8 [N, K / block * block_bytes]."""
    blocks: torch.Tensor
    ggml_type: int
    k: int
    bias: Optional[torch.Tensor] = None

    is_fp8 = False        # so that model code can treat it like a LinearWeight
    is_mx = False

    @property
    def out_features(self) -> int:
        return self.blocks.shape[0]

    @property
    def in_features(self) -> int:
        return self.k

    def nbytes(self) -> int:
        return self.blocks.numel() + (0 if self.bias is None else self.bias.numel() * 2)

    @staticmethod
    def supported(ggml_type: int, k: int) -> bool:
        return ggml_type in _GGUF_ROW and k % _GGUF_ROW[ggml_type][0] == 0

    @staticmethod
    def from_raw(raw: torch.Tensor, ggml_type: int, n: int, k: int, bias: Optional[torch.Tensor] = None) -> "GgufWeight":
        per, nbytes = _GGUF_ROW[ggml_type]
        return GgufWeight(raw.reshape(n, k // per * nbytes), ggml_type, k, bias)

    def dequantize(self) -> torch.Tensor:
        """bf16 [N, K] (device kernel on CUDA, host codec on CPU)."""
        n = self.blocks.shape[0]
        if not self.blocks.is_cuda:
            from ..assets.gguf import dequantize
            return dequantize(self.blocks.contiguous(), self.ggml_type, n * self.k).reshape(n, self.k).to(torch.bfloat16)
        out = torch.empty(n, self.k, dtype=torch.bfloat16, device=self.blocks.device)
        rc = N.lib().b200_gguf_dequant(self.blocks.data_ptr(), self.ggml_type, out.data_ptr(), n, self.k, N.stream())
        N.check(rc, "b200_gguf_dequant")
        return out


def gguf_linear(x: torch.Tensor, w: GgufWeight, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x @ W^T + bias with W read as ggml blocks: up to 16 tokens go through the integer-dot
    GEMV (each weight bit read once), more tokens dequantise to a bf16 scratch and use the GEMM."""
    m, k = x.shape
    assert k == w.k
    if not x.is_cuda:
        y = x.float() @ w.dequantize().float().t()
        if w.bias is not None:
            y = y + w.bias.float()
        return y.to(x.dtype)
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1 and w.blocks.is_contiguous()
    n = w.out_features
    if m > GGUF_GEMV_MAX_TOKENS:
        return linear(x, LinearWeight(w.dequantize(), None, w.bias), out=out)
    if out is None:
        out = torch.empty(m, n, dtype=torch.bfloat16, device=x.device)
    L = N.lib()
    ws = torch.empty(L.b200_gguf_gemv_workspace_bytes(m, k), dtype=torch.uint8, device=x.device)
    rc = L.b200_gguf_gemv(x.data_ptr(), x.stride(0), w.blocks.data_ptr(), w.ggml_type, out.data_ptr(), out.stride(0),
                          N.ptr(w.bias), m, n, k, ws.data_ptr(), N.stream())
    N.check(rc, "b200_gguf_gemv")
    return out


# ---------------------------------------------------------------------------------------------
# convolution as one shifted-row GEMM (no im2col buffer)
# ---------------------------------------------------------------------------------------------
def pack_conv3d_weight(weight: torch.Tensor) -> torch.Tensor:
    """[Cout, Cin, kt, kh, kw] -> bf16 [Cout, kt * kh * kw * Cin_p] with taps outermost and the
    channel count padded to a multiple of 64 (done once per weight)."""
    co, ci, kt, kh, kw = weight.shape
    cp = (ci + 63) // 64 * 64
    w = torch.zeros(co, kt, kh, kw, cp, dtype=torch.bfloat16, device=weight.device)
    w[..., :ci] = weight.permute(0, 2, 3, 4, 1).to(torch.bfloat16)
    return w.reshape(co, kt * kh * kw * cp).contiguous()


def causal_conv3d(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                  packed: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Stride-1 3-D convolution, "same" padding in H and W, causal in T (kt - 1 zero frames in
    front). x [C, T, H, W] or [1, C, T, H, W]; weight [Cout, Cin, kt, kh, kw]. On the device this
    is one tcgen05 GEMM over the zero-padded channels-last volume: tap (dt, dy, dx) is the same
    [positions, Cin] matrix shifted down by (dt * Hp + dy) * Wp + dx rows."""
    batched = x.dim() == 5
    if batched:
        assert x.shape[0] == 1
        x = x[0]
    co, ci, kt, kh, kw = weight.shape
    c, t, h, w_ = x.shape
    assert c == ci
    if not x.is_cuda:
        xp = torch.nn.functional.pad(x[None].float(), (kw // 2, kw // 2, kh // 2, kh // 2, kt - 1, 0))
        y = torch.nn.functional.conv3d(xp, weight.float(), None if bias is None else bias.float())[0].to(x.dtype)
        return y[None] if batched else y
    cp = (ci + 63) // 64 * 64
    tp, hp, wp = t + kt - 1, h + kh - 1, w_ + kw - 1
    xp = torch.zeros(tp, hp, wp, cp, dtype=torch.bfloat16, device=x.device)
    xp[kt - 1:, kh // 2:kh // 2 + h, kw // 2:kw // 2 + w_, :ci] = x.permute(1, 2, 3, 0)
    if packed is None:
        packed = pack_conv3d_weight(weight)
    shifts = torch.tensor([(dt * hp + dy) * wp + dx for dt in range(kt) for dy in range(kh) for dx in range(kw)],
                          dtype=torch.int32)
    rows = t * hp * wp
    out = torch.empty(rows, co, dtype=torch.bfloat16, device=x.device)
    st = N.state(x.device)
    ws = st.gemm_workspace()
    bias_b = None if bias is None else bias.to(torch.bfloat16).contiguous()
    rc = N.lib().b200_conv_gemm(xp.data_ptr(), tp * hp * wp, cp, packed.data_ptr(), co, kt * kh * kw,
                                shifts.data_ptr(), out.data_ptr(), rows, co, N.ptr(bias_b), 0, ws.data_ptr(),
                                ws.numel(), st.status.data_ptr(), N.stream())
    N.check(rc, "b200_conv_gemm")
    y = out.view(t, hp, wp, co)[:, :h, :w_, :].permute(3, 0, 1, 2).contiguous().to(x.dtype)
    return y[None] if batched else y


# ---------------------------------------------------------------------------------------------
# state-space scan
# ---------------------------------------------------------------------------------------------
def selective_scan(x: torch.Tensor, dt: torch.Tensor, a: torch.Tensor, b: torch.Tensor, c: torch.Tensor,
                   d: torch.Tensor, state: torch.Tensor) -> torch.Tensor:
    """Mamba selective scan on the device: x [T, Di] bf16, dt [T, Di] fp32, a [Di, N] fp32 (negative),
    b / c [T, N] bf16, d [Di] fp32, state [Di, N] fp32 (updated in place). Returns y [T, Di] bf16."""
    t, di = x.shape
    n = a.shape[1]
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous() and dt.dtype == torch.float32
    assert dt.is_contiguous() and a.is_contiguous() and state.is_contiguous() and state.dtype == torch.float32
    b = b.to(torch.bfloat16).contiguous()
    c = c.to(torch.bfloat16).contiguous()
    y = torch.empty(t, di, dtype=torch.bfloat16, device=x.device)
    rc = N.lib().b200_selective_scan(x.data_ptr(), dt.data_ptr(), a.data_ptr(), b.data_ptr(), c.data_ptr(),
                                     d.data_ptr(), state.data_ptr(), y.data_ptr(), t, di, n, N.stream())
    N.check(rc, "b200_selective_scan")
    return y
