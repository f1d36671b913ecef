"""Plain PyTorch fp32 statements of every op: the numerical oracle of the CUDA kernels and the
implementation used for CPU tensors.

The reference engine keeps the same idea: every ``IBackend`` op has a CPU default body that the
accelerated backends are tested against (src/HartsyInference.Core/Backends/IBackend.cs,
src/HartsyInference.Core/Backends/AttentionReference.cs). Nothing here is tuned for speed.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

FP8_MAX = 448.0


# --------------------------------------------------------------------------------------------
# quantisation
# --------------------------------------------------------------------------------------------
def pow2_scale(amax: torch.Tensor) -> torch.Tensor:
    """Smallest power of two >= amax / 448 (UE8M0 scale), exponent clamped to [-126, 126]."""
    m, ex = torch.frexp(amax.float() / FP8_MAX)          # value = m * 2^ex, m in [0.5, 1)
    e = torch.where(m == 0.5, ex - 1, ex).clamp(-126, 126)
    return torch.ldexp(torch.ones_like(m), e)


def pack_sf(scale: torch.Tensor, tile_rows: int = 128) -> torch.Tensor:
    """Power-of-two scales [rows, K/128] -> the blocked UE8M0 layout of the block-scaled GEMM:
    int32 [row tiles, ceil(K/512), 128]; a tile covers ``tile_rows`` (<= 128) rows, row r of a tile
    sits at word (r % 32) * 4 + r // 32 and K block kb at byte kb % 4 of the word."""
    rows, kb = scale.shape
    e = (torch.log2(scale.float()).round().to(torch.int32) + 127).clamp(0, 254).to(torch.uint8)
    kg = (kb + 3) // 4
    tiles = (rows + tile_rows - 1) // tile_rows
    ep = torch.full((rows, kg * 4), 127, dtype=torch.uint8, device=scale.device)
    ep[:, :kb] = e
    out = torch.full((tiles, kg, 128, 4), 127, dtype=torch.uint8, device=scale.device)
    r = torch.arange(rows, device=scale.device)
    tile, rr = r // tile_rows, r % tile_rows
    out[tile, :, (rr % 32) * 4 + rr // 32, :] = ep.reshape(rows, kg, 4)
    return out.view(torch.int32).reshape(tiles, kg, 128)


def unpack_sf(sf: torch.Tensor, rows: int, kb: int, tile_rows: int = 128) -> torch.Tensor:
    """Inverse of :func:`pack_sf`: fp32 scales [rows, kb]."""
    tiles, kg, _ = sf.shape
    b = sf.contiguous().view(torch.uint8).reshape(tiles, kg, 128, 4)
    r = torch.arange(rows, device=sf.device)
    tile, rr = r // tile_rows, r % tile_rows
    e = b[tile, :, (rr % 32) * 4 + rr // 32, :].reshape(rows, kg * 4)[:, :kb]
    return torch.ldexp(torch.ones(rows, kb, device=sf.device), e.to(torch.int32) - 127)


def quant_fp8_act(x: torch.Tensor, pow2: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    """1x128 block quantisation of activations [M, K] -> (e4m3 bytes [M, K], scales [M, K/128])."""
    m, k = x.shape
    assert k % 128 == 0
    xf = x.float().reshape(m, k // 128, 128)
    amax = xf.abs().amax(dim=-1).clamp_min(1e-12)
    scale = pow2_scale(amax) if pow2 else amax / FP8_MAX
    q = (xf / scale.unsqueeze(-1)).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q.reshape(m, k).view(torch.uint8), scale.contiguous()


def quant_fp8_weight(w: torch.Tensor, pow2: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    """128x128 block quantisation of a weight [N, K] -> (bytes [N, K], scales [ceil(N/128), K/128])."""
    n, k = w.shape
    assert k % 128 == 0
    nb = (n + 127) // 128
    wf = torch.zeros(nb * 128, k, dtype=torch.float32, device=w.device)
    wf[:n] = w.float()
    blocks = wf.reshape(nb, 128, k // 128, 128)
    amax = blocks.abs().amax(dim=(1, 3)).clamp_min(1e-12)       # [nb, kb]
    scale = pow2_scale(amax) if pow2 else amax / FP8_MAX
    q = (blocks / scale[:, None, :, None]).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    q = q.reshape(nb * 128, k)[:n]
    return q.contiguous().view(torch.uint8), scale.contiguous()


def dequant_fp8_act(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    m, k = q.shape
    f = q.view(torch.float8_e4m3fn).float().reshape(m, k // 128, 128)
    return (f * scale.unsqueeze(-1)).reshape(m, k)


def dequant_fp8_weight(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    n, k = q.shape
    s = scale.repeat_interleave(128, dim=0)[:n].repeat_interleave(128, dim=1)
    return q.view(torch.float8_e4m3fn).float() * s


# --------------------------------------------------------------------------------------------
# linear
# --------------------------------------------------------------------------------------------
def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    return torch.nn.functional.gelu(x, approximate="tanh")


def linear(x: torch.Tensor, w: torch.Tensor, w_scale: Optional[torch.Tensor] = None,
           x_scale: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
           act: Optional[str] = None, gate: Optional[torch.Tensor] = None,
           residual: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """y = residual + gate * act(x @ w^T + bias); fp8 operands are dequantised first."""
    xf = dequant_fp8_act(x, x_scale) if x_scale is not None else x.float()
    wf = dequant_fp8_weight(w, w_scale) if w_scale is not None else w.float()
    y = xf @ wf.t()
    if bias is not None:
        y = y + bias.float()
    if act == "gelu_tanh":
        y = gelu_tanh(y)
    elif act == "silu":
        y = torch.nn.functional.silu(y)
    if gate is not None:
        y = y * gate.float()
    if residual is not None:
        y = y + residual.float()
    return y.to(out_dtype)


# --------------------------------------------------------------------------------------------
# norms / activations
# --------------------------------------------------------------------------------------------
def norm(x: torch.Tensor, weight: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
         residual: Optional[torch.Tensor] = None, shift: Optional[torch.Tensor] = None,
         scale: Optional[torch.Tensor] = None, rows_per_batch: int = 0, eps: float = 1e-6,
         layernorm: bool = False, weight_plus_one: bool = False):
    """Returns (y fp32, h) where h = x + residual rounded to the storage dtype (or None)."""
    h = x.float()
    h_out = None
    if residual is not None:
        h = (h + residual.float()).to(x.dtype)
        h_out = h
        h = h.float()
    if layernorm:
        mean = h.mean(dim=-1, keepdim=True)
        var = ((h - mean) ** 2).mean(dim=-1, keepdim=True)
        y = (h - mean) * torch.rsqrt(var + eps)
    else:
        y = h * torch.rsqrt((h * h).mean(dim=-1, keepdim=True) + eps)
    if weight is not None:
        w = weight.float()
        y = y * ((1.0 + w) if weight_plus_one else w)
    if bias is not None:
        y = y + bias.float()
    if scale is not None or shift is not None:
        rows = y.shape[0]
        rpb = rows_per_batch if rows_per_batch > 0 else rows
        idx = torch.arange(rows, device=y.device) // rpb
        if scale is not None:
            y = y * (1.0 + scale.float()[idx][:, : y.shape[1]])
        if shift is not None:
            y = y + shift.float()[idx][:, : y.shape[1]]
    return y, h_out


def glu(x: torch.Tensor, act: str = "silu") -> torch.Tensor:
    f = x.shape[-1] // 2
    g, u = x[..., :f].float(), x[..., f:].float()
    a = torch.nn.functional.silu(g) if act == "silu" else gelu_tanh(g)
    return a * u


# --------------------------------------------------------------------------------------------
# rotary embedding
# --------------------------------------------------------------------------------------------
def rope_inv_freq(rot: int, theta: float, device=None) -> torch.Tensor:
    return theta ** (-torch.arange(0, rot, 2, dtype=torch.float32, device=device) / rot)


def apply_rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, style: int = 0) -> torch.Tensor:
    """x [T, H, D]; rotates the first 2 * len(inv_freq) dims. style 0 = split-half, 1 = interleaved."""
    rot = inv_freq.numel() * 2
    xf = x.float()
    ang = positions.float()[:, None] * inv_freq[None, :]          # [T, rot/2]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    xr, rest = xf[..., :rot], xf[..., rot:]
    if style == 0:
        a, b = xr[..., : rot // 2], xr[..., rot // 2:]
        out = torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)
    else:
        a, b = xr[..., 0::2], xr[..., 1::2]
        out = torch.stack([a * cos - b * sin, b * cos + a * sin], dim=-1).flatten(-2)
    return torch.cat([out, rest], dim=-1)


# --------------------------------------------------------------------------------------------
# attention
# --------------------------------------------------------------------------------------------
def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = False,
              scale: Optional[float] = None, softcap: float = 0.0, window: int = 0,
              alibi: Optional[torch.Tensor] = None, sinks: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q [Tq, Hq, D], k/v [Tk, Hkv, D] (one sequence). The last query row sits at key position
    Tk - 1 (so a query chunk with a cached prefix is expressed by Tk > Tq). ``alibi`` [Hq] adds
    slope * key position to the scores; ``sinks`` [Hq] adds one extra logit per head to the softmax
    denominator (it attends to nothing). Returns fp32 [Tq, Hq, D]."""
    tq, hq, d = q.shape
    tk, hkv, _ = k.shape
    g = hq // hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    kf = k.float().repeat_interleave(g, dim=1)
    vf = v.float().repeat_interleave(g, dim=1)
    s = torch.einsum("qhd,khd->hqk", q.float(), kf) * scale
    if softcap > 0:
        s = softcap * torch.tanh(s / softcap)
    qpos = torch.arange(tq, device=q.device)[:, None] + (tk - tq)
    kpos = torch.arange(tk, device=q.device)[None, :]
    mask = torch.ones(tq, tk, dtype=torch.bool, device=q.device)
    if causal:
        mask &= kpos <= qpos
    if window > 0:
        mask &= kpos > qpos - window
    if alibi is not None:
        s = s + alibi.float()[:, None, None] * kpos[None].float()
    s = s.masked_fill(~mask[None], float("-inf"))
    if sinks is not None:
        s = torch.cat([s, sinks.float()[:, None, None].expand(hq, tq, 1)], -1)
    p = torch.softmax(s, dim=-1)
    p = torch.nan_to_num(p)
    if sinks is not None:
        p = p[..., :tk]
    return torch.einsum("hqk,khd->qhd", p, vf)


def gather_paged(cache: torch.Tensor, table: torch.Tensor, length: int) -> torch.Tensor:
    """cache [pages, Hkv, page, D], table [max_pages] -> [length, Hkv, D]."""
    page = cache.shape[2]
    n = (length + page - 1) // page
    pages = cache[table[:n].long()]                               # [n, Hkv, page, D]
    return pages.permute(0, 2, 1, 3).reshape(n * page, cache.shape[1], cache.shape[3])[:length]


# --------------------------------------------------------------------------------------------
# diffusion scheduler step
# --------------------------------------------------------------------------------------------
def cfg_euler(z: torch.Tensor, cond: torch.Tensor, uncond: Optional[torch.Tensor], g: float, dt: float) -> torch.Tensor:
    v = cond.float() if uncond is None else g * cond.float() + (1.0 - g) * uncond.float()
    return z + v * dt


# --------------------------------------------------------------------------------------------
# mixture of experts
# --------------------------------------------------------------------------------------------
def moe_route(logits: torch.Tensor, bias: Optional[torch.Tensor], top_k: int, n_group: int = 1,
              topk_group: int = 1, sigmoid: bool = False, norm_topk: bool = False,
              scale: float = 1.0) -> tuple[torch.Tensor, torch.Tensor]:
    """Top-k routing. Returns (expert ids int32 [T, k], mixing weights fp32 [T, k]).

    Softmax or sigmoid scores; optional DeepSeek-V3 group-limited selection (selection score =
    score + bias, group score = sum of the group's two best, keep ``topk_group`` groups); the
    weight is the unbiased score, renormalised when ``norm_topk`` and multiplied by ``scale``.
    Ties go to the lower expert index."""
    lg = logits.float()
    t, e = lg.shape
    score = torch.sigmoid(lg) if sigmoid else torch.softmax(lg, dim=-1)
    sel = score + bias.float() if bias is not None else score.clone()
    if n_group > 1 and topk_group < n_group:
        g = sel.view(t, n_group, e // n_group)
        gscore = g.topk(min(2, e // n_group), dim=-1).values.sum(-1)
        keep = torch.zeros(t, n_group, dtype=torch.bool, device=lg.device)
        work = gscore.clone()
        for _ in range(topk_group):
            idx = work.argmax(dim=-1, keepdim=True)     # first maximum = lowest index
            keep.scatter_(1, idx, True)
            work.scatter_(1, idx, float("-inf"))
        sel = sel.masked_fill(~keep.unsqueeze(-1).expand(t, n_group, e // n_group).reshape(t, e), float("-inf"))
    ids = torch.empty(t, top_k, dtype=torch.int64, device=lg.device)
    work = sel.clone()
    for r in range(top_k):
        idx = work.argmax(dim=-1)
        ids[:, r] = idx
        work.scatter_(1, idx.unsqueeze(1), float("-inf"))
    w = score.gather(1, ids)
    if norm_topk:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return ids.to(torch.int32), w * scale


def sampling_keep_mask(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, min_p: float) -> torch.Tensor:
    """Tokens that survive temperature -> top-k -> top-p -> min-p for one row of fp32 logits, with
    ties at a cut kept (the statement the device sampler is checked against). Returns a bool mask."""
    lg = logits.float() / max(temperature, 1e-6)
    w = torch.exp(lg - lg.max())
    keep = torch.ones_like(w, dtype=torch.bool)
    if 0 < top_k < w.numel():
        kth = torch.topk(w, top_k).values[-1]
        keep &= w >= kth
    if 0.0 < top_p < 1.0:
        ws = torch.where(keep, w, torch.zeros_like(w))
        sp, _ = torch.sort(ws, descending=True)
        cum = torch.cumsum(sp.double(), 0)
        limit = top_p * float(ws.double().sum())
        first_over = int((cum > limit).nonzero()[0]) if bool((cum > limit).any()) else w.numel() - 1
        keep &= w >= sp[first_over]
    if min_p > 0.0:
        keep &= w >= min(min_p, 1.0)
    return keep


def msda(value: torch.Tensor, shapes: list, offsets: torch.Tensor, logits: torch.Tensor, ref: torch.Tensor) -> torch.Tensor:
    """Multi-scale deformable attention between its linear layers, fp32.

    value [B, S, heads, D] (levels concatenated along S in the order of ``shapes`` = [(h, w), ...]),
    offsets [B, Q, heads, L, P, 2], logits [B, Q, heads, L, P], ref [B, Q, 4] (cx, cy, w, h), [B, Q, 2]
    or per level [B, Q, L, 2 | 4]. Softmax over the L * P points, locations as in Deformable DETR
    (4-d: centre + offset / P * size / 2; 2-d: point + offset / (w, h) of the level), bilinear
    samples with zero padding and pixel centres at half-integers. Returns [B, Q, heads * D]."""
    b, s_, heads, d = value.shape
    _, q, _, lv, pts, _ = offsets.shape
    v = value.float()
    w = torch.softmax(logits.float().reshape(b, q, heads, lv * pts), -1).reshape(b, q, heads, lv, pts)
    r = ref.float()
    if r.dim() == 3:
        r = r[:, :, None, :].expand(b, q, lv, r.shape[-1])
    out = torch.zeros(b, q, heads, d)
    out = out.to(v.device)
    start = 0
    for li, (h, wd) in enumerate(shapes):
        vl = v[:, start:start + h * wd].reshape(b, h, wd, heads, d)
        start += h * wd
        off = offsets[:, :, :, li].float()                               # [B, Q, heads, P, 2]
        rl = r[:, :, li]                                                 # [B, Q, 2 | 4]
        if rl.shape[-1] == 4:
            loc = rl[:, :, None, None, :2] + off / pts * rl[:, :, None, None, 2:] * 0.5
        else:
            loc = rl[:, :, None, None, :] + off / torch.tensor([wd, h], dtype=torch.float32, device=v.device)
        x = loc[..., 0] * wd - 0.5
        y = loc[..., 1] * h - 0.5
        x0, y0 = torch.floor(x), torch.floor(y)
        ax, ay = x - x0, y - y0
        bi = torch.arange(b, device=v.device)[:, None, None, None]
        hi = torch.arange(heads, device=v.device)[None, None, :, None]
        for dy in (0, 1):
            for dx in (0, 1):
                xx, yy = (x0 + dx).long(), (y0 + dy).long()
                ok = (xx >= 0) & (xx < wd) & (yy >= 0) & (yy < h)
                cw = (ax if dx else 1 - ax) * (ay if dy else 1 - ay) * w[:, :, :, li] * ok
                g = vl[bi, yy.clamp(0, h - 1), xx.clamp(0, wd - 1), hi]  # [B, Q, heads, P, D]
                out += (cw[..., None] * g).sum(3)
    return out.reshape(b, q, heads * d)


def cfg_renorm_euler(z: torch.Tensor, cond: torch.Tensor, uncond: torch.Tensor, guidance: float, dt: float,
                     renorm_min: float = 0.0) -> torch.Tensor:
    """z + s * guided * dt with guided = uncond + g (cond - uncond) and one scale for the whole tensor,
    s = clamp(||cond|| / (||guided|| + 1e-8), renorm_min, 1) (norms in double precision)."""
    c, u = cond.double(), uncond.double()
    guided = (uncond.float() + guidance * (cond.float() - uncond.float()))
    ratio = float(c.pow(2).sum().sqrt() / (guided.double().pow(2).sum().sqrt() + 1e-8))
    ratio = renorm_min if ratio < renorm_min else 1.0 if ratio > 1.0 else ratio
    return z.float() + guided * (ratio * dt)


def cfg_rownorm_euler(z: torch.Tensor, cond: torch.Tensor, uncond: torch.Tensor, guidance: float, dt: float,
                      eps: float = 1e-12) -> torch.Tensor:
    """The same with one ratio per row of the last dimension and no clamp; a zero denominator gives 0."""
    guided = uncond.float() + guidance * (cond.float() - uncond.float())
    den = guided.double().pow(2).sum(-1, keepdim=True).sqrt() + eps
    ratio = torch.where(den > 0, cond.double().pow(2).sum(-1, keepdim=True).sqrt() / den, torch.zeros_like(den)).float()
    return z.float() + guided * ratio * dt
