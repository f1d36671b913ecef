"""Grounding DINO: open-set detection from a picture and a text of phrases ("a cat . a remote control .").

* picture: Swin backbone -> the last three maps through 1 x 1 convolution + GroupNorm to 256
  channels, plus a fourth level from a stride-2 3 x 3 convolution; sine position codes (temperature
  20) + a learned code per level;
* text: BERT run with phrase-wise attention (tokens see only the tokens between the same pair of
  separators ``[CLS] [SEP] . ?``) and positions restarting after every separator, projected to 256;
* encoder layer x 6: (a) fusion: LayerNorm both streams, picture queries over text keys and the
  transposed scores for text over picture, shared score matrix, outputs scaled by learned
  per-channel factors and added to the NORMED streams; (b) text self-attention with sine positions
  under the phrase mask + feed-forward; (c) multi-scale deformable self-attention over the four
  levels (one kernel: ``ops.msda``) + feed-forward;
* queries: every encoder position proposes a box (its cell centre, 0.05 x 2^level wide); positions
  are ranked by their best similarity to a text token and the top ``num_queries`` become the
  reference boxes, the queries themselves are learned embeddings;
* decoder layer x 6: self-attention, cross-attention to the text, deformable cross-attention to
  the picture around the reference box, feed-forward; after every layer the box is refined in
  logit space; class scores are dot products of the (normed) query with the text states.

Weights by the `transformers` names (``model.backbone.conv_encoder.model.*``, ``model.text_backbone.*``,
``model.encoder.*``, ``model.decoder.*``, ``bbox_embed.*``). Reference:
src/HartsyInference.Vision/Detection/GroundingDino/, Kernels/vision/msda.cu.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.nn.functional as F

from ... import ops
from ..encoders.swin import SwinBackbone, SwinConfig

SEPARATORS = (101, 102, 1012, 1029)          # [CLS] [SEP] . ?  in the BERT uncased vocabulary


@dataclass(frozen=True)
class GroundingDinoConfig:
    d_model: int = 256
    encoder_layers: int = 6
    decoder_layers: int = 6
    heads: int = 8
    encoder_ffn: int = 2048
    decoder_ffn: int = 2048
    levels: int = 4
    enc_points: int = 4
    dec_points: int = 4
    num_queries: int = 900
    max_text_len: int = 256
    eps: float = 1e-5
    temperature: float = 20.0
    text_hidden: int = 768
    text_layers: int = 12
    text_heads: int = 12
    text_eps: float = 1e-12
    share_box_heads: bool = True
    swin: SwinConfig = SwinConfig()

    @staticmethod
    def from_hf(d: dict) -> "GroundingDinoConfig":
        t, b = d.get("text_config", {}), d.get("backbone_config", {})
        return GroundingDinoConfig(d_model=d.get("d_model", 256), encoder_layers=d.get("encoder_layers", 6), decoder_layers=d.get("decoder_layers", 6),
                                   heads=d.get("encoder_attention_heads", 8), encoder_ffn=d.get("encoder_ffn_dim", 2048),
                                   decoder_ffn=d.get("decoder_ffn_dim", 2048), levels=d.get("num_feature_levels", 4),
                                   enc_points=d.get("encoder_n_points", 4), dec_points=d.get("decoder_n_points", 4),
                                   num_queries=d.get("num_queries", 900), max_text_len=d.get("max_text_len", 256), eps=d.get("layer_norm_eps", 1e-5),
                                   temperature=d.get("positional_embedding_temperature", 20.0), text_hidden=t.get("hidden_size", 768),
                                   text_layers=t.get("num_hidden_layers", 12), text_heads=t.get("num_attention_heads", 12),
                                   text_eps=t.get("layer_norm_eps", 1e-12), share_box_heads=bool(d.get("decoder_bbox_embed_share", True)),
                                   swin=SwinConfig.from_hf(b))


def phrase_masks(ids: torch.Tensor, separators=SEPARATORS):
    """ids [L] -> (allowed [L, L] bool: tokens between the same separators see each other, everyone sees
    itself; positions [L] restarting after each separator)."""
    n = ids.numel()
    special = torch.isin(ids, torch.tensor(separators, device=ids.device))
    idx = torch.arange(n, device=ids.device)
    prev = torch.cummax(torch.where(special, idx, torch.full_like(idx, -1)), 0)[0]
    nxt = torch.flip(torch.cummin(torch.flip(torch.where(special, idx, torch.full_like(idx, n)), [0]), 0)[0], [0])
    valid = (nxt != 0) & (nxt != n - 1) & (nxt != n)
    allowed = ((nxt[:, None] == nxt[None, :]) & valid[None, :]) | torch.eye(n, dtype=torch.bool, device=ids.device)
    pos = torch.where(valid, idx - prev - 1, torch.zeros_like(idx)).clamp(min=0)
    return allowed, pos


def sine_embed(values: torch.Tensor, feats: int, temperature: float = 10000.0, swap_xy: bool = True) -> torch.Tensor:
    """values [..., k] in [0, 1] -> [..., k * feats]: interleaved sin / cos per coordinate (y before x when asked)."""
    dim_t = temperature ** (2 * torch.div(torch.arange(feats, dtype=torch.float32, device=values.device), 2, rounding_mode="floor") / feats)
    parts = []
    for i in range(values.shape[-1]):
        s = values[..., i, None] * (2 * math.pi) / dim_t
        parts.append(torch.stack((s[..., 0::2].sin(), s[..., 1::2].cos()), -1).flatten(-2))
    if swap_xy and len(parts) >= 2:
        parts[0], parts[1] = parts[1], parts[0]
    return torch.cat(parts, -1)


class GroundingDino:
    def __init__(self, cfg: GroundingDinoConfig, get: Callable[[str], Optional[torch.Tensor]], device="cpu", dtype: torch.dtype = torch.float32):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        self._get, self._cache = get, {}
        self.backbone = SwinBackbone(cfg.swin, get, device, dtype, prefix="model.backbone.conv_encoder.model.")

    # ------------------------------------------------------------------------------ helpers
    def _w(self, name: str, optional: bool = False):
        hit = self._cache.get(name, False)
        if hit is False:
            t = self._get(name)
            if t is None and not optional:
                raise KeyError(name)
            hit = None if t is None else t.to(self.device).to(self.dtype)
            self._cache[name] = hit
        return hit

    def _lin(self, x, p: str):
        return F.linear(x, self._w(p + ".weight"), self._w(p + ".bias", True))

    def _ln(self, x, p: str, eps: Optional[float] = None):
        return F.layer_norm(x, (x.shape[-1],), self._w(p + ".weight"), self._w(p + ".bias"), self.cfg.eps if eps is None else eps)

    def _mlp(self, x, p: str, n: int):
        for i in range(n):
            x = self._lin(x, f"{p}.layers.{i}")
            if i < n - 1:
                x = F.relu(x)
        return x

    def _mha(self, q, k, v, p: str, heads: int, mask: Optional[torch.Tensor] = None):
        b, lq, c = q.shape
        d = c // heads
        split = lambda t: t.view(b, -1, heads, d).transpose(1, 2)
        o = F.scaled_dot_product_attention(split(self._lin(q, p + ".query")), split(self._lin(k, p + ".key")), split(self._lin(v, p + ".value")),
                                           attn_mask=mask)
        return self._lin(o.transpose(1, 2).reshape(b, lq, c), p + ".out_proj")

    def _deformable(self, query, memory, ref, shapes, p: str, points: int):
        """query [B, Q, C] (positions added), memory [B, S, C], ref [B, Q, L, 2 | 4] -> [B, Q, C]."""
        cfg = self.cfg
        b, q, c = query.shape
        value = self._lin(memory, p + ".value_proj").view(b, memory.shape[1], cfg.heads, c // cfg.heads)
        offsets = self._lin(query, p + ".sampling_offsets").view(b, q, cfg.heads, cfg.levels, points, 2)
        logits = self._lin(query, p + ".attention_weights").view(b, q, cfg.heads, cfg.levels, points)
        out = ops.msda(value.contiguous(), shapes, offsets.float(), logits.float(), ref.float().contiguous())
        return self._lin(out.to(query.dtype), p + ".output_proj")

    # ------------------------------------------------------------------------------ text
    @torch.no_grad()
    def text_states(self, ids: torch.Tensor):
        """ids [L] -> (BERT states projected to d_model [1, L, C], allowed [L, L], positions [L])."""
        cfg = self.cfg
        ids = ids.to(self.device).long()[:cfg.max_text_len]
        allowed, pos = phrase_masks(ids)
        p = "model.text_backbone."
        x = self._w(p + "embeddings.word_embeddings.weight")[ids] + self._w(p + "embeddings.position_embeddings.weight")[pos] \
            + self._w(p + "embeddings.token_type_embeddings.weight")[torch.zeros_like(ids)]
        x = self._ln(x, p + "embeddings.LayerNorm", cfg.text_eps)[None]
        d = cfg.text_hidden // cfg.text_heads
        split = lambda t: t.view(1, -1, cfg.text_heads, d).transpose(1, 2)
        for i in range(cfg.text_layers):
            q_ = f"{p}encoder.layer.{i}."
            a = F.scaled_dot_product_attention(split(self._lin(x, q_ + "attention.self.query")), split(self._lin(x, q_ + "attention.self.key")),
                                               split(self._lin(x, q_ + "attention.self.value")), attn_mask=allowed)
            x = self._ln(x + self._lin(a.transpose(1, 2).reshape(1, -1, cfg.text_hidden), q_ + "attention.output.dense"),
                         q_ + "attention.output.LayerNorm", cfg.text_eps)
            x = self._ln(x + self._lin(F.gelu(self._lin(x, q_ + "intermediate.dense")), q_ + "output.dense"), q_ + "output.LayerNorm", cfg.text_eps)
        return self._lin(x, "model.text_projection"), allowed, pos

    # ------------------------------------------------------------------------------ picture
    def _position_codes(self, h: int, w: int) -> torch.Tensor:
        cfg = self.cfg
        half = cfg.d_model // 2
        y = torch.arange(1, h + 1, dtype=torch.float32, device=self.device) / (h + 1e-6) * (2 * math.pi)
        x = torch.arange(1, w + 1, dtype=torch.float32, device=self.device) / (w + 1e-6) * (2 * math.pi)
        dim_t = cfg.temperature ** (2 * torch.div(torch.arange(half, dtype=torch.float32, device=self.device), 2, rounding_mode="floor") / half)
        enc = lambda v: torch.stack(((v[:, None] / dim_t)[:, 0::2].sin(), (v[:, None] / dim_t)[:, 1::2].cos()), -1).flatten(1)
        py, px = enc(y), enc(x)                                          # [h, half], [w, half]
        return torch.cat([py[:, None].expand(h, w, half), px[None].expand(h, w, half)], -1).reshape(h * w, cfg.d_model)

    @torch.no_grad()
    def picture_levels(self, pixels: torch.Tensor):
        """pixels [1, 3, H, W] -> (flattened levels [1, S, C], position + level codes [1, S, C], shapes)."""
        cfg = self.cfg
        maps = self.backbone(pixels)
        levels = []
        for i, m in enumerate(maps):
            y = F.conv2d(m, self._w(f"model.input_proj_vision.{i}.0.weight"), self._w(f"model.input_proj_vision.{i}.0.bias"))
            levels.append(F.group_norm(y, 32, self._w(f"model.input_proj_vision.{i}.1.weight"), self._w(f"model.input_proj_vision.{i}.1.bias")))
        for i in range(len(maps), cfg.levels):
            src = maps[-1] if i == len(maps) else levels[-1]
            y = F.conv2d(src, self._w(f"model.input_proj_vision.{i}.0.weight"), self._w(f"model.input_proj_vision.{i}.0.bias"), stride=2, padding=1)
            levels.append(F.group_norm(y, 32, self._w(f"model.input_proj_vision.{i}.1.weight"), self._w(f"model.input_proj_vision.{i}.1.bias")))
        shapes = [tuple(l.shape[-2:]) for l in levels]
        flat = torch.cat([l.flatten(2).transpose(1, 2) for l in levels], 1)
        codes = torch.cat([self._position_codes(h, w).to(self.dtype) + self._w("model.level_embed")[i] for i, (h, w) in enumerate(shapes)], 0)[None]
        return flat, codes, shapes

    # ------------------------------------------------------------------------------ all of it
    @torch.no_grad()
    def forward(self, pixels: torch.Tensor, ids: torch.Tensor):
        """pixels [1, 3, H, W] (ImageNet-normalised), ids [L] (BERT ids of "[CLS] phrase . phrase . [SEP]") ->
        (logits [Q, L]: similarity of every query to every text token, boxes [Q, 4] as cx, cy, w, h in [0, 1])."""
        cfg = self.cfg
        c, heads = cfg.d_model, cfg.heads
        text, allowed, pos = self.text_states(ids)
        vision, codes, shapes = self.picture_levels(pixels.to(self.device).to(self.dtype))
        n_text = text.shape[1]
        refs = []
        for h, w in shapes:
            ys, xs = torch.meshgrid((torch.arange(h, device=self.device) + 0.5) / h, (torch.arange(w, device=self.device) + 0.5) / w, indexing="ij")
            refs.append(torch.stack([xs.reshape(-1), ys.reshape(-1)], -1))
        enc_ref = torch.cat(refs, 0)[None, :, None].expand(1, -1, cfg.levels, 2).float()
        text_pos = sine_embed(pos[None, :, None].float(), c, swap_xy=False).to(self.dtype)
        fh = heads // 2
        for i in range(cfg.encoder_layers):
            p = f"model.encoder.layers.{i}."
            # (a) fusion
            v, t = self._ln(vision, p + "fusion_layer.layer_norm_vision"), self._ln(text, p + "fusion_layer.layer_norm_text")
            a = p + "fusion_layer.attn."
            e = self._w(a + "vision_proj.weight").shape[0]
            d = e // fh
            split = lambda u: u.view(1, -1, fh, d).transpose(1, 2)
            vq, tk = split(self._lin(v, a + "vision_proj") * d ** -0.5), split(self._lin(t, a + "text_proj"))
            vv, tv = split(self._lin(v, a + "values_vision_proj")), split(self._lin(t, a + "values_text_proj"))
            scores = vq @ tk.transpose(-1, -2)                                        # [1, fh, S, L]
            scores = (scores - scores.max()).clamp(-50000, 50000)
            st = scores.transpose(-1, -2)
            st = (st - st.max(-1, keepdim=True)[0]).clamp(-50000, 50000)
            dv = self._lin((scores.softmax(-1) @ tv).transpose(1, 2).reshape(1, -1, e), a + "out_vision_proj")
            dt = self._lin((st.softmax(-1) @ vv).transpose(1, 2).reshape(1, -1, e), a + "out_text_proj")
            vision = v + self._w(p + "fusion_layer.vision_param") * dv
            text = t + self._w(p + "fusion_layer.text_param") * dt
            # (b) text
            e_ = p + "text_enhancer_layer."
            qk = text + text_pos
            text = self._ln(text + self._mha(qk, qk, text, e_ + "self_attn", fh, allowed), e_ + "layer_norm_before")
            text = self._ln(text + self._lin(F.relu(self._lin(text, e_ + "fc1")), e_ + "fc2"), e_ + "layer_norm_after")
            # (c) picture
            d_ = p + "deformable_layer."
            vision = self._ln(vision + self._deformable(vision + codes, vision, enc_ref, shapes, d_ + "self_attn", cfg.enc_points),
                              d_ + "self_attn_layer_norm")
            vision = self._ln(vision + self._lin(F.relu(self._lin(vision, d_ + "fc1")), d_ + "fc2"), d_ + "final_layer_norm")
        # ---- proposals and query selection
        props = []
        for lvl, (h, w) in enumerate(shapes):
            ys, xs = torch.meshgrid((torch.arange(h, device=self.device) + 0.5) / h, (torch.arange(w, device=self.device) + 0.5) / w, indexing="ij")
            wh = torch.full((h * w, 2), 0.05 * 2.0 ** lvl, device=self.device)
            props.append(torch.cat([xs.reshape(-1, 1), ys.reshape(-1, 1), wh], -1))
        props = torch.cat(props, 0)[None]
        ok = ((props > 0.01) & (props < 0.99)).all(-1, keepdim=True)
        prop_logits = torch.log(props / (1 - props)).masked_fill(~ok, float("inf"))
        memory = self._ln(self._lin(vision.masked_fill(~ok, 0.0), "model.enc_output"), "model.enc_output_norm")
        sim = memory @ text.transpose(-1, -2)                                         # [1, S, L]
        top = sim.max(-1)[0].topk(min(cfg.num_queries, sim.shape[1]), 1)[1]
        coords = self._mlp(memory, "model.encoder_output_bbox_embed", 3).float() + prop_logits
        ref = coords.gather(1, top[..., None].expand(-1, -1, 4)).sigmoid()
        nq = ref.shape[1]
        hidden = self._w("model.query_position_embeddings.weight")[None, :nq]
        # ---- decoder
        out_logits = out_boxes = None
        for i in range(cfg.decoder_layers):
            p = f"model.decoder.layers.{i}."
            ref_in = ref[:, :, None].expand(-1, -1, cfg.levels, -1)
            qpos = self._mlp(sine_embed(ref_in[:, :, 0], c // 2).to(self.dtype), "model.decoder.reference_points_head", 2)
            qk = hidden + qpos
            hidden = self._ln(hidden + self._mha(qk, qk, hidden, p + "self_attn", heads), p + "self_attn_layer_norm")
            hidden = self._ln(hidden + self._mha(hidden + qpos, text, text, p + "encoder_attn_text", heads), p + "encoder_attn_text_layer_norm")
            hidden = self._ln(hidden + self._deformable(hidden + qpos, vision, ref_in, shapes, p + "encoder_attn", cfg.dec_points),
                              p + "encoder_attn_layer_norm")
            hidden = self._ln(hidden + self._lin(F.relu(self._lin(hidden, p + "fc1")), p + "fc2"), p + "final_layer_norm")
            head = f"bbox_embed.{i}" if self._w(f"bbox_embed.{i}.layers.0.weight", True) is not None else "bbox_embed.0"
            normed = self._ln(hidden, "model.decoder.layer_norm")
            prev = torch.special.logit(ref, eps=1e-5)
            # the layer's output box: its own head on the NORMED state; the next reference: the head on the raw state
            out_boxes = (self._mlp(normed, head, 3).float() + prev).sigmoid()
            out_logits = normed @ text.transpose(-1, -2)
            ref = (self._mlp(hidden, head, 3).float() + prev).sigmoid()
        return out_logits[0].float(), out_boxes[0].float()

    @torch.no_grad()
    def detect(self, pixels: torch.Tensor, ids: torch.Tensor, box_threshold: float = 0.35, text_threshold: float = 0.25) -> list:
        """-> [(token positions of the matched phrase, score, (cx, cy, w, h))], best first."""
        logits, boxes = self.forward(pixels, ids)
        probs = logits.sigmoid()
        best = probs.max(-1)[0]
        keep = (best > box_threshold).nonzero().flatten()
        keep = keep[best[keep].argsort(descending=True)]
        return [((probs[i] > text_threshold).nonzero().flatten().tolist(), float(best[i]), tuple(boxes[i].tolist())) for i in keep.tolist()]
