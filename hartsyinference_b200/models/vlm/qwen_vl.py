"""Qwen2-VL / Qwen2.5-VL: the (windowed) vision transformer, its 2x2 patch merger, and the three-axis rotary
positions (M-RoPE) its decoder uses.

Vision tower, for one image of ``gh x gw`` patches (both even):
    patches [gh * gw, 3 * 2 * p * p] in merge-block order (the four patches of each 2x2 block are
    consecutive) -> linear patch embedding -> ``depth`` blocks of RMSNorm, attention with a 2-D
    rotary embedding (first half of the rotary dims from the patch row, second half from its column),
    RMSNorm, SwiGLU MLP. Blocks listed in ``full_blocks`` attend over the whole image; the others
    only within windows of ``window / patch / merge`` merged cells per side. The merger normalises,
    concatenates each 2x2 block and maps it through a two-layer MLP to the decoder width.

Qwen2-VL's tower is the same skeleton with LayerNorm, a plain quick-GELU MLP and full attention in
every block (``QwenVisionConfig.legacy``).

Attention inside a window is expressed with a block mask on the natural token order, so no
reordering (and no inverse reordering after the merger) is needed.
Reference: src/HartsyInference.Core/Multimodal/ (Qwen2.5-VL encoder, Qwen35VlGenerator).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional, Sequence

import torch
import torch.nn.functional as F


@dataclass(frozen=True)
class QwenVisionConfig:
    hidden: int = 1280
    heads: int = 16
    ffn: int = 3420
    depth: int = 32
    out_hidden: int = 3584
    patch: int = 14
    temporal_patch: int = 2
    merge: int = 2
    window: int = 112
    full_blocks: tuple = (7, 15, 23, 31)
    eps: float = 1e-6
    legacy: bool = False                # Qwen2-VL: LayerNorm, plain quick-GELU MLP, full attention in every block

    @staticmethod
    def from_hf(d: dict) -> "QwenVisionConfig":
        if d.get("model_type") == "qwen2_vl" or "embed_dim" in d:
            hidden = d.get("embed_dim", 1280)
            return QwenVisionConfig(hidden=hidden, heads=d.get("num_heads", 16), ffn=int(hidden * d.get("mlp_ratio", 4)),
                                    depth=d.get("depth", 32), out_hidden=d.get("hidden_size", 3584), patch=d.get("patch_size", 14),
                                    temporal_patch=d.get("temporal_patch_size", 2), merge=d.get("spatial_merge_size", 2),
                                    window=0, full_blocks=(), legacy=True)
        return QwenVisionConfig(hidden=d.get("hidden_size", 1280), heads=d.get("num_heads", 16), ffn=d.get("intermediate_size", 3420),
                                depth=d.get("depth", 32), out_hidden=d.get("out_hidden_size", 3584), patch=d.get("patch_size", 14),
                                temporal_patch=d.get("temporal_patch_size", 2), merge=d.get("spatial_merge_size", 2),
                                window=d.get("window_size", 112), full_blocks=tuple(d.get("fullatt_block_indexes") or (7, 15, 23, 31)))


def _rms(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)


def merge_block_coords(gh: int, gw: int, merge: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Row and column of every patch in merge-block order ([gh * gw] each)."""
    rows = torch.arange(gh)[:, None].expand(gh, gw).reshape(gh // merge, merge, gw // merge, merge).permute(0, 2, 1, 3).flatten()
    cols = torch.arange(gw)[None, :].expand(gh, gw).reshape(gh // merge, merge, gw // merge, merge).permute(0, 2, 1, 3).flatten()
    return rows, cols


def patchify(image: torch.Tensor, cfg, max_pixels: int = 1280 * 28 * 28) -> tuple[torch.Tensor, int, int]:
    """image [3, H, W] in [0, 1] -> (patches [gh * gw, 3 * temporal * p * p] in merge-block order, gh, gw).
    The image is resized to multiples of ``patch * merge``, CLIP-normalised and repeated along time."""
    from ..encoders.clip_vision import CLIP_MEAN, CLIP_STD
    p, m, tp = cfg.patch, cfg.merge, cfg.temporal_patch
    unit = p * m
    _, h, w = image.shape
    scale = min(1.0, (max_pixels / (h * w)) ** 0.5)
    hh, ww = max(unit, round(h * scale / unit) * unit), max(unit, round(w * scale / unit) * unit)
    x = F.interpolate(image[None].float(), size=(hh, ww), mode="bicubic", align_corners=False, antialias=True)[0].clamp(0, 1)
    if isinstance(cfg, Qwen3VisionConfig):                    # Qwen3-VL normalises to [-1, 1]
        x = (x - 0.5) / 0.5
    else:
        x = (x - torch.tensor(CLIP_MEAN).view(3, 1, 1)) / torch.tensor(CLIP_STD).view(3, 1, 1)
    gh, gw = hh // p, ww // p
    x = x[None].expand(tp, 3, hh, ww).reshape(tp, 3, gh // m, m, p, gw // m, m, p)
    x = x.permute(2, 5, 3, 6, 1, 0, 4, 7)                     # block row, block col, in-block row, in-block col, C, T, p, p
    return x.reshape(gh * gw, 3 * tp * p * p).contiguous(), gh, gw


def _norm(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    if b is None:
        return _rms(x, w, eps)
    return F.layer_norm(x.float(), (x.shape[-1],), w.float(), b.float(), eps).to(x.dtype)


class _Block:
    def __init__(self, t: Callable, p: str, legacy: bool = False):
        self.n1, self.n2 = t(p + "norm1.weight"), t(p + "norm2.weight")
        self.n1_b = self.n2_b = None
        self.qkv_w, self.qkv_b = t(p + "attn.qkv.weight"), t(p + "attn.qkv.bias")
        self.proj_w, self.proj_b = t(p + "attn.proj.weight"), t(p + "attn.proj.bias")
        self.legacy = legacy
        if legacy:
            self.n1_b, self.n2_b = t(p + "norm1.bias"), t(p + "norm2.bias")
            self.fc1_w, self.fc1_b, self.fc2_w, self.fc2_b = t(p + "mlp.fc1.weight"), t(p + "mlp.fc1.bias"), t(p + "mlp.fc2.weight"), t(p + "mlp.fc2.bias")
            return
        self.gate_w, self.gate_b = t(p + "mlp.gate_proj.weight"), t(p + "mlp.gate_proj.bias")
        self.up_w, self.up_b = t(p + "mlp.up_proj.weight"), t(p + "mlp.up_proj.bias")
        self.down_w, self.down_b = t(p + "mlp.down_proj.weight"), t(p + "mlp.down_proj.bias")

    def __call__(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, mask: Optional[torch.Tensor], heads: int, eps: float):
        n, c = x.shape
        d = c // heads
        q, k, v = F.linear(_norm(x, self.n1, self.n1_b, eps), self.qkv_w, self.qkv_b).reshape(n, 3, heads, d).unbind(1)

        def rot(u):
            uf = u.float()
            u1, u2 = uf[..., : d // 2], uf[..., d // 2:]
            return (uf * cos[:, None] + torch.cat([-u2, u1], -1) * sin[:, None]).to(u.dtype)

        a = F.scaled_dot_product_attention(rot(q).transpose(0, 1)[None], rot(k).transpose(0, 1)[None], v.transpose(0, 1)[None],
                                           attn_mask=mask)[0]
        x = x + F.linear(a.transpose(0, 1).reshape(n, c), self.proj_w, self.proj_b)
        h = _norm(x, self.n2, self.n2_b, eps)
        if self.legacy:
            u = F.linear(h, self.fc1_w, self.fc1_b)
            return x + F.linear(u * torch.sigmoid(1.702 * u.float()).to(u.dtype), self.fc2_w, self.fc2_b)
        return x + F.linear(F.silu(F.linear(h, self.gate_w, self.gate_b)) * F.linear(h, self.up_w, self.up_b), self.down_w, self.down_b)


class QwenVisionTower:
    def __init__(self, cfg: QwenVisionConfig, get: Callable[[str], Optional[torch.Tensor]], device="cpu",
                 dtype: torch.dtype = torch.bfloat16, prefix: str = "model.visual."):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype

        def t(n):
            w = get(prefix + n)
            if w is None:
                raise KeyError(f"missing tensor {prefix + n}")
            return w.to(dtype).to(self.device)

        self.patch_w = t("patch_embed.proj.weight").reshape(cfg.hidden, -1)
        self.blocks = [_Block(t, f"blocks.{i}.", cfg.legacy) for i in range(cfg.depth)]
        self.ln_q = t("merger.ln_q.weight")
        self.ln_q_b = t("merger.ln_q.bias") if cfg.legacy else None
        self.m0_w, self.m0_b, self.m2_w, self.m2_b = t("merger.mlp.0.weight"), t("merger.mlp.0.bias"), t("merger.mlp.2.weight"), t("merger.mlp.2.bias")
        d = cfg.hidden // cfg.heads
        self.inv_freq = 1.0 / (10000.0 ** (torch.arange(0, d // 2, 2, dtype=torch.float32) / (d // 2)))

    @torch.no_grad()
    def __call__(self, patches: torch.Tensor, gh: int, gw: int) -> torch.Tensor:
        """patches [gh * gw, 3 * temporal * p * p] (merge-block order) -> [gh * gw / merge^2, out_hidden]."""
        cfg = self.cfg
        x = F.linear(patches.to(self.device, self.dtype), self.patch_w)
        rows, cols = merge_block_coords(gh, gw, cfg.merge)
        fr = torch.cat([rows[:, None].float() * self.inv_freq[None], cols[:, None].float() * self.inv_freq[None]], -1)
        emb = torch.cat([fr, fr], -1).to(self.device)
        cos, sin = emb.cos(), emb.sin()
        wmask = None
        if cfg.window > 0:
            cells = cfg.window // cfg.merge // cfg.patch                     # window side in merged cells
            win = ((rows // cfg.merge) // cells) * (gw // cfg.merge // cells + 1) + (cols // cfg.merge) // cells
            wmask = (win[:, None] == win[None, :]).to(self.device)
        for i, blk in enumerate(self.blocks):
            x = blk(x, cos, sin, None if (i in cfg.full_blocks or wmask is None) else wmask, cfg.heads, cfg.eps)
        g = cfg.merge * cfg.merge
        y = _norm(x, self.ln_q, self.ln_q_b, cfg.eps).reshape(-1, g * cfg.hidden)
        return F.linear(F.gelu(F.linear(y, self.m0_w, self.m0_b)), self.m2_w, self.m2_b)


@dataclass(frozen=True)
class Qwen3VisionConfig:
    hidden: int = 1152
    heads: int = 16
    ffn: int = 4304
    depth: int = 27
    out_hidden: int = 3584
    patch: int = 16
    temporal_patch: int = 2
    merge: int = 2
    num_positions: int = 2304
    deepstack: tuple = (8, 16, 24)
    eps: float = 1e-6
    window: int = 0

    @staticmethod
    def from_hf(d: dict) -> "Qwen3VisionConfig":
        return Qwen3VisionConfig(hidden=d.get("hidden_size", 1152), heads=d.get("num_heads", 16), ffn=d.get("intermediate_size", 4304),
                                 depth=d.get("depth", 27), out_hidden=d.get("out_hidden_size", 3584), patch=d.get("patch_size", 16),
                                 temporal_patch=d.get("temporal_patch_size", 2), merge=d.get("spatial_merge_size", 2),
                                 num_positions=d.get("num_position_embeddings", 2304),
                                 deepstack=tuple(d.get("deepstack_visual_indexes") or ()))


class _Merger3:
    """LayerNorm (before or after the 2x2 blocks are concatenated) -> Linear -> GELU -> Linear."""

    def __init__(self, t: Callable, p: str, post_shuffle: bool):
        self.nw, self.nb = t(p + "norm.weight"), t(p + "norm.bias")
        self.w1, self.b1, self.w2, self.b2 = t(p + "linear_fc1.weight"), t(p + "linear_fc1.bias"), t(p + "linear_fc2.weight"), t(p + "linear_fc2.bias")
        self.post_shuffle = post_shuffle

    def __call__(self, x: torch.Tensor, group: int, eps: float) -> torch.Tensor:
        wide = x.shape[-1] * group
        y = _norm(x.reshape(-1, wide), self.nw, self.nb, eps) if self.post_shuffle else _norm(x, self.nw, self.nb, eps).reshape(-1, wide)
        return F.linear(F.gelu(F.linear(y, self.w1, self.b1)), self.w2, self.b2)


class Qwen3VisionTower:
    """Qwen3-VL tower: patch embedding with bias + a learned position table interpolated bilinearly to
    the image's grid, LayerNorm / tanh-GELU blocks with the 2-D rotary embedding and full attention,
    the merger, and "deepstack" mergers that tap the blocks in ``cfg.deepstack``; their outputs are
    added to the decoder's hidden states at the image rows after its first layers."""

    def __init__(self, cfg: Qwen3VisionConfig, get: Callable[[str], Optional[torch.Tensor]], device="cpu",
                 dtype: torch.dtype = torch.bfloat16, prefix: str = "model.visual."):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype

        def t(n):
            w = get(prefix + n)
            if w is None:
                raise KeyError(f"missing tensor {prefix + n}")
            return w.to(dtype).to(self.device)

        self.patch_w, self.patch_b = t("patch_embed.proj.weight").reshape(cfg.hidden, -1), t("patch_embed.proj.bias")
        self.pos = t("pos_embed.weight")
        self.blocks = []
        for i in range(cfg.depth):
            p = f"blocks.{i}."
            self.blocks.append(dict(n1=t(p + "norm1.weight"), n1b=t(p + "norm1.bias"), n2=t(p + "norm2.weight"), n2b=t(p + "norm2.bias"),
                                    qkv=t(p + "attn.qkv.weight"), qkvb=t(p + "attn.qkv.bias"), proj=t(p + "attn.proj.weight"),
                                    projb=t(p + "attn.proj.bias"), f1=t(p + "mlp.linear_fc1.weight"), f1b=t(p + "mlp.linear_fc1.bias"),
                                    f2=t(p + "mlp.linear_fc2.weight"), f2b=t(p + "mlp.linear_fc2.bias")))
        self.merger = _Merger3(t, "merger.", False)
        self.deep = [_Merger3(t, f"deepstack_merger_list.{i}.", True) for i in range(len(cfg.deepstack))]
        d = cfg.hidden // cfg.heads
        self.inv_freq = 1.0 / (10000.0 ** (torch.arange(0, d // 2, 2, dtype=torch.float32) / (d // 2)))

    def _positions(self, gh: int, gw: int) -> torch.Tensor:
        """The side x side position table sampled bilinearly on a gh x gw grid, in merge-block order."""
        side = int(self.cfg.num_positions ** 0.5)
        hi, wi = torch.linspace(0, side - 1, gh), torch.linspace(0, side - 1, gw)
        h0, w0 = hi.int(), wi.int()
        h1, w1 = (h0 + 1).clamp(max=side - 1), (w0 + 1).clamp(max=side - 1)
        dh, dw = (hi - h0)[:, None], (wi - w0)[None, :]
        tab = self.pos.float().cpu()
        at = lambda a, b: tab[(a[:, None] * side + b[None, :]).long().flatten()].reshape(gh, gw, -1)
        out = (at(h0, w0) * ((1 - dh) * (1 - dw))[..., None] + at(h0, w1) * ((1 - dh) * dw)[..., None]
               + at(h1, w0) * (dh * (1 - dw))[..., None] + at(h1, w1) * (dh * dw)[..., None])
        m = self.cfg.merge
        out = out.reshape(gh // m, m, gw // m, m, -1).permute(0, 2, 1, 3, 4).reshape(gh * gw, -1)
        return out.to(self.dtype).to(self.device)

    @torch.no_grad()
    def __call__(self, patches: torch.Tensor, gh: int, gw: int) -> tuple[torch.Tensor, list[torch.Tensor]]:
        """-> (merged tokens [gh * gw / merge^2, out_hidden], one tensor of the same shape per deepstack tap)."""
        cfg = self.cfg
        x = F.linear(patches.to(self.device, self.dtype), self.patch_w, self.patch_b) + self._positions(gh, gw)
        rows, cols = merge_block_coords(gh, gw, cfg.merge)
        fr = torch.cat([rows[:, None].float() * self.inv_freq[None], cols[:, None].float() * self.inv_freq[None]], -1)
        emb = torch.cat([fr, fr], -1).to(self.device)
        cos, sin = emb.cos()[:, None], emb.sin()[:, None]
        n, c = x.shape
        d = c // cfg.heads
        g = cfg.merge * cfg.merge

        def rot(u):
            uf = u.float()
            return (uf * cos + torch.cat([-uf[..., d // 2:], uf[..., : d // 2]], -1) * sin).to(u.dtype)

        taps = []
        for i, b in enumerate(self.blocks):
            q, k, v = F.linear(_norm(x, b["n1"], b["n1b"], cfg.eps), b["qkv"], b["qkvb"]).reshape(n, 3, cfg.heads, d).unbind(1)
            a = F.scaled_dot_product_attention(rot(q).transpose(0, 1)[None], rot(k).transpose(0, 1)[None], v.transpose(0, 1)[None])[0]
            x = x + F.linear(a.transpose(0, 1).reshape(n, c), b["proj"], b["projb"])
            h = _norm(x, b["n2"], b["n2b"], cfg.eps)
            x = x + F.linear(F.gelu(F.linear(h, b["f1"], b["f1b"]), approximate="tanh"), b["f2"], b["f2b"])
            if i in cfg.deepstack:
                taps.append(self.deep[cfg.deepstack.index(i)](x, g, cfg.eps))
        return self.merger(x, g, cfg.eps), taps


def mrope_positions(ids: Sequence[int], image_token_id: int, grids: Sequence[tuple[int, int]]) -> tuple[torch.Tensor, int]:
    """Three-axis positions [3, len(ids)] (time, row, column) and the offset to add to the sequence
    index for every token generated afterwards. Text advances all three axes together; the tokens
    of an image (``grids`` gives each image's merged rows x columns) share one time index and
    spread over rows and columns; the text after it continues from the largest index used."""
    out, cur, i, k = [], 0, 0, 0
    n = len(ids)
    while i < n:
        if ids[i] == image_token_id and k < len(grids):
            r, c = grids[k]
            k += 1
            t = torch.full((r * c,), cur, dtype=torch.int64)
            hh = torch.arange(cur, cur + r).repeat_interleave(c)
            ww = torch.arange(cur, cur + c).repeat(r)
            out.append(torch.stack([t, hh, ww]))
            cur += max(r, c)
            i += r * c
        else:
            j = i
            while j < n and not (ids[j] == image_token_id and k < len(grids)):
                j += 1
            out.append((torch.arange(j - i) + cur)[None].expand(3, -1))
            cur += j - i
            i = j
    pos = torch.cat(out, 1)
    return pos.to(torch.int32), int(pos.max()) + 1 - n


class QwenVlModel:
    """Decoder + vision tower. ``expand_prompt`` turns a prompt with one image token per image into
    (ids, embeds, mask, positions3, rope_delta) for the engine; a Qwen3-VL tower also leaves the
    deepstack rows of that prompt in ``self.deepstack`` ([taps, len(ids), hidden], else None)."""

    three_axis_positions = True
    deepstack: Optional[torch.Tensor] = None

    def __init__(self, decoder, cfg, get: Callable[[str], Optional[torch.Tensor]], image_token_id: int,
                 prefix: str = "model.visual.", vision_start_id: Optional[int] = None, vision_end_id: Optional[int] = None):
        self.decoder, self.image_token_id = decoder, image_token_id
        self.image_prefix_ids = () if vision_start_id is None else (int(vision_start_id),)
        self.image_suffix_ids = () if vision_end_id is None else (int(vision_end_id),)
        tower = Qwen3VisionTower if isinstance(cfg, Qwen3VisionConfig) else QwenVisionTower
        self.vision = tower(cfg, get, decoder.device, torch.bfloat16, prefix)

    def image_features(self, image: torch.Tensor) -> tuple[torch.Tensor, int, int, list]:
        """(merged tokens, merged rows, merged columns, deepstack taps)."""
        patches, gh, gw = patchify(image, self.vision.cfg)
        m = self.vision.cfg.merge
        out = self.vision(patches, gh, gw)
        feats, taps = out if isinstance(out, tuple) else (out, [])
        return feats, gh // m, gw // m, taps

    def expand_prompt(self, ids: Sequence[int], images: Sequence[torch.Tensor]):
        feats = [self.image_features(im) for im in images]
        out: list[int] = []
        rows: list[torch.Tensor] = []
        k = 0
        for tok in ids:
            if tok == self.image_token_id and k < len(feats):
                out.extend([tok] * feats[k][0].shape[0])
                rows.append(feats[k][0])
                k += 1
            else:
                out.append(tok)
        if k != len(feats):
            raise ValueError(f"{len(feats)} image(s) for {k} image token(s) in the prompt")
        mask = torch.tensor([t == self.image_token_id for t in out])
        hidden = self.decoder.cfg.hidden_size
        embeds = torch.zeros(len(out), hidden, dtype=torch.bfloat16, device=self.decoder.device)
        if rows:
            embeds[mask.to(embeds.device)] = torch.cat(rows, 0).to(embeds.dtype)
        pos3, delta = mrope_positions(out, self.image_token_id, [(r, c) for _, r, c, _ in feats])
        self.deepstack = None
        if feats and feats[0][3]:
            # [taps, len(ids), hidden]: every tap's tokens at the image rows, zero at the text rows
            self.deepstack = torch.zeros(len(feats[0][3]), len(out), hidden, dtype=torch.bfloat16, device=self.decoder.device)
            for li in range(self.deepstack.shape[0]):
                self.deepstack[li][mask.to(embeds.device)] = torch.cat([f[3][li] for f in feats], 0).to(torch.bfloat16)
        return out, embeds, mask, pos3, delta
