"""SAM 2 promptable image segmentation (Hiera backbone, feature pyramid, prompt encoder, mask decoder).

* backbone: 7x7 stride-4 patch convolution, a position table (a small background grid resampled
  bicubically to the feature map + a window-sized table tiled over it), then four stages of blocks.
  A block is LayerNorm -> attention -> residual -> LayerNorm -> MLP -> residual; attention runs inside
  non-overlapping windows except in a few global blocks; the first block of stages 2-4 widens the
  channels and max-pools the queries 2x2 (so the map shrinks and its residual is pooled too);
* neck: 1x1 convolutions to one width, coarse-to-fine, with nearest-neighbour top-down addition on the
  configured levels, and a normalised 2-d sine position code per level;
* prompts: points and box corners become random-Fourier position codes plus a learned type vector;
  a given mask is embedded by two stride-2 convolutions (otherwise one learned "no mask" vector);
* mask decoder: object-score, IoU and mask tokens + prompt tokens go through a two-way transformer
  (token self-attention, token->image and image->token cross-attention with halved inner width), the
  image side is upsampled 4x by two transposed convolutions that add the two finer pyramid levels, and
  every mask token's hyper-network MLP gives the filter that turns the upsampled features into one mask.

Image segmentation only (the video memory bank is not part of this module). Reference:
src/HartsyInference.Vision/Segmentation/ (SAM 2 behind the vision service's segment operation).
Tensor names follow Hugging Face ``Sam2Model``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, Optional

import torch
import torch.nn.functional as F


@dataclass
class Sam2Config:
    # backbone
    image_size: int = 1024
    patch_kernel: int = 7
    patch_stride: int = 4
    patch_padding: int = 3
    query_stride: int = 2
    background_size: tuple = (7, 7)
    num_query_pool_stages: int = 3
    blocks_per_stage: tuple = (1, 2, 7, 2)
    embed_dims: tuple = (96, 192, 384, 768)
    heads_per_stage: tuple = (1, 2, 4, 8)
    window_sizes: tuple = (8, 4, 14, 7)
    global_blocks: tuple = (5, 7, 9)
    mlp_ratio: float = 4.0
    backbone_eps: float = 1e-6
    # neck
    fpn_dim: int = 256
    fpn_top_down_levels: tuple = (2, 3)
    num_feature_levels: int = 3
    # prompt encoder
    prompt_image_size: int = 1024
    prompt_patch: int = 16
    mask_input_channels: int = 16
    prompt_eps: float = 1e-6
    # mask decoder
    hidden: int = 256
    decoder_mlp_dim: int = 2048
    decoder_layers: int = 2
    decoder_heads: int = 8
    attention_downsample: int = 2
    num_multimask_outputs: int = 3
    iou_head_hidden: int = 256
    iou_head_depth: int = 3
    dynamic_multimask: bool = True
    stability_delta: float = 0.05
    stability_thresh: float = 0.98


def sam2_from_hf(d: dict) -> Sam2Config:
    v = d.get("vision_config") or {}
    b = v.get("backbone_config") or {}
    p = d.get("prompt_encoder_config") or {}
    m = d.get("mask_decoder_config") or {}
    first = lambda x, dflt: (x[0] if isinstance(x, (list, tuple)) else x) if x is not None else dflt
    return Sam2Config(
        image_size=first(b.get("image_size"), 1024), patch_kernel=first(b.get("patch_kernel_size"), 7),
        patch_stride=first(b.get("patch_stride"), 4), patch_padding=first(b.get("patch_padding"), 3),
        query_stride=first(b.get("query_stride"), 2),
        background_size=tuple(b.get("window_positional_embedding_background_size", (7, 7))),
        num_query_pool_stages=b.get("num_query_pool_stages", 3), blocks_per_stage=tuple(b.get("blocks_per_stage", (1, 2, 7, 2))),
        embed_dims=tuple(b.get("embed_dim_per_stage", (96, 192, 384, 768))),
        heads_per_stage=tuple(b.get("num_attention_heads_per_stage", (1, 2, 4, 8))),
        window_sizes=tuple(b.get("window_size_per_stage", (8, 4, 14, 7))), global_blocks=tuple(b.get("global_attention_blocks", (5, 7, 9))),
        mlp_ratio=float(b.get("mlp_ratio", 4.0)), backbone_eps=float(b.get("layer_norm_eps", 1e-6)),
        fpn_dim=v.get("fpn_hidden_size", 256), fpn_top_down_levels=tuple(v.get("fpn_top_down_levels", (2, 3))),
        num_feature_levels=v.get("num_feature_levels", 3), prompt_image_size=p.get("image_size", 1024),
        prompt_patch=p.get("patch_size", 16), mask_input_channels=p.get("mask_input_channels", 16),
        prompt_eps=float(p.get("layer_norm_eps", 1e-6)), hidden=m.get("hidden_size", 256), decoder_mlp_dim=m.get("mlp_dim", 2048),
        decoder_layers=m.get("num_hidden_layers", 2), decoder_heads=m.get("num_attention_heads", 8),
        attention_downsample=m.get("attention_downsample_rate", 2), num_multimask_outputs=m.get("num_multimask_outputs", 3),
        iou_head_hidden=m.get("iou_head_hidden_dim", 256), iou_head_depth=m.get("iou_head_depth", 3),
        dynamic_multimask=bool(m.get("dynamic_multimask_via_stability", True)),
        stability_delta=float(m.get("dynamic_multimask_stability_delta", 0.05)),
        stability_thresh=float(m.get("dynamic_multimask_stability_thresh", 0.98)))


def _windows(x: torch.Tensor, ws: int):
    """[B, H, W, C] -> ([B * nW, ws, ws, C], padded (H, W))."""
    b, h, w, c = x.shape
    ph, pw = (ws - h % ws) % ws, (ws - w % ws) % ws
    x = F.pad(x, (0, 0, 0, pw, 0, ph))
    hp, wp = h + ph, w + pw
    x = x.view(b, hp // ws, ws, wp // ws, ws, c).permute(0, 1, 3, 2, 4, 5).reshape(-1, ws, ws, c)
    return x, (hp, wp)


def _unwindows(x: torch.Tensor, ws: int, padded: tuple, hw: tuple) -> torch.Tensor:
    hp, wp = padded
    b = x.shape[0] // (hp * wp // ws // ws)
    x = x.view(b, hp // ws, wp // ws, ws, ws, -1).permute(0, 1, 3, 2, 4, 5).reshape(b, hp, wp, -1)
    return x[:, :hw[0], :hw[1]].contiguous()


def _pool(x: torch.Tensor, k: int) -> torch.Tensor:
    return F.max_pool2d(x.permute(0, 3, 1, 2), k, k).permute(0, 2, 3, 1)


class Sam2:
    """``get(name)`` returns checkpoint tensors by their Hugging Face names. Inference only."""

    def __init__(self, cfg: Sam2Config, device="cpu", get: Optional[Callable[[str], Optional[torch.Tensor]]] = None,
                 dtype: Optional[torch.dtype] = None):
        if get is None:
            raise ValueError("SAM 2 needs a checkpoint")
        self.cfg, self.device = cfg, torch.device(device)
        self.dtype = dtype or (torch.bfloat16 if self.device.type == "cuda" else torch.float32)
        self._get, self._w = get, {}

    # ------------------------------------------------------------------------------ weights / small ops
    def _t(self, name: str, optional: bool = False):
        t = self._w.get(name)
        if t is None:
            raw = self._get(name)
            if raw is None:
                if optional:
                    return None
                raise KeyError(name)
            t = raw.to(self.device).to(self.dtype)
            self._w[name] = t
        return t

    def _lin(self, x, p: str):
        return F.linear(x, self._t(p + ".weight"), self._t(p + ".bias", optional=True))

    def _ln(self, x, p: str, eps: float):
        return F.layer_norm(x, (x.shape[-1],), self._t(p + ".weight"), self._t(p + ".bias"), eps)

    def _ln2d(self, x, p: str, eps: float = 1e-6):
        return self._ln(x.permute(0, 2, 3, 1), p, eps).permute(0, 3, 1, 2)

    def _conv(self, x, p: str, stride: int = 1, padding: int = 0):
        return F.conv2d(x, self._t(p + ".weight"), self._t(p + ".bias", optional=True), stride=stride, padding=padding)

    def _ffn(self, x, p: str, layers: int, act=F.relu, sigmoid: bool = False):
        x = act(self._lin(x, p + ".proj_in"))
        for i in range(layers - 2):
            x = act(self._lin(x, f"{p}.layers.{i}"))
        x = self._lin(x, p + ".proj_out")
        return torch.sigmoid(x) if sigmoid else x

    # ------------------------------------------------------------------------------ backbone + neck
    def _block(self, x, index: int, stage: int, first: bool):
        cfg = self.cfg
        p = f"vision_encoder.backbone.blocks.{index}"
        dim_in = cfg.embed_dims[stage - 1] if (stage > 0 and first) else cfg.embed_dims[stage]
        dim_out, heads = cfg.embed_dims[stage], cfg.heads_per_stage[stage]
        ws = cfg.window_sizes[stage - 1] if (stage > 0 and first) else cfg.window_sizes[stage]
        if index in cfg.global_blocks:
            ws = 0
        stride = cfg.query_stride if (0 < stage <= cfg.num_query_pool_stages and first) else 0
        res = x
        y = self._ln(x, p + ".layer_norm1", cfg.backbone_eps)
        if dim_in != dim_out:
            res = _pool(self._lin(y, p + ".proj"), stride) if stride else self._lin(y, p + ".proj")
        hh, ww = y.shape[1], y.shape[2]
        padded = (hh, ww)
        if ws > 0:
            y, padded = _windows(y, ws)
        b, h, w, _ = y.shape
        qkv = self._lin(y, p + ".attn.qkv").reshape(b, h * w, 3, heads, dim_out // heads)
        q, k, v = qkv.unbind(2)
        if stride:
            q = _pool(q.reshape(b, h, w, dim_out), stride)
            h, w = q.shape[1:3]
            q = q.reshape(b, h * w, heads, dim_out // heads)
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)).transpose(1, 2)
        y = self._lin(o.reshape(b, h, w, dim_out), p + ".attn.proj")
        if stride:
            ws = ws // stride
            hh, ww = res.shape[1:3]
            padded = (hh + (ws - hh % ws) % ws, ww + (ws - ww % ws) % ws) if ws > 0 else (hh, ww)
        if ws > 0:
            y = _unwindows(y, ws, padded, (hh, ww))
        x = res + y
        return x + self._ffn(self._ln(x, p + ".layer_norm2", cfg.backbone_eps), p + ".mlp", 2, act=F.gelu)

    def _position_table(self, h: int, w: int):
        bg = self._t("vision_encoder.backbone.pos_embed").float()
        win = self._t("vision_encoder.backbone.pos_embed_window").float()
        pos = F.interpolate(bg, size=(h, w), mode="bicubic")
        pos = pos + win.tile([1, 1, h // win.shape[2], w // win.shape[3]])
        return pos.permute(0, 2, 3, 1).to(self.dtype)

    @torch.no_grad()
    def image_embeddings(self, pixels: torch.Tensor) -> list:
        """pixels [B, 3, S, S] normalised -> pyramid [fine (already reduced to hidden / 8 channels), middle
        (hidden / 4), coarse (hidden, with the no-memory vector added)], each [B, C, h, w]."""
        cfg = self.cfg
        x = self._conv(pixels.to(self.device).to(self.dtype), "vision_encoder.backbone.patch_embed.projection", cfg.patch_stride,
                       cfg.patch_padding).permute(0, 2, 3, 1)
        x = x + self._position_table(x.shape[1], x.shape[2])
        stage_out, index = [], 0
        for stage, n in enumerate(cfg.blocks_per_stage):
            for bi in range(n):
                x = self._block(x, index, stage, bi == 0)
                index += 1
            stage_out.append(x)
        n = len(stage_out) - 1
        maps, prev = [], None
        for i in range(n, -1, -1):                                    # coarse to fine
            lat = self._conv(stage_out[i].permute(0, 3, 1, 2), f"vision_encoder.neck.convs.{n - i}")
            if i not in cfg.fpn_top_down_levels or i == n:
                prev = lat
            else:
                prev = lat + F.interpolate(prev.float(), scale_factor=2.0, mode="nearest").to(lat.dtype)
            maps.append(prev)
        maps = maps[-cfg.num_feature_levels:][::-1]                   # fine ... coarse
        maps[0] = self._conv(maps[0], "mask_decoder.conv_s0")
        maps[1] = self._conv(maps[1], "mask_decoder.conv_s1")
        maps[-1] = maps[-1] + self._t("no_memory_embedding").reshape(1, -1, 1, 1)
        return maps

    # ------------------------------------------------------------------------------ prompts
    def _fourier(self, coords: torch.Tensor) -> torch.Tensor:
        """coords [..., 2] in [0, 1] -> [..., hidden] random-Fourier position code."""
        g = self._t("shared_image_embedding.positional_embedding").float()
        c = (2 * coords.float() - 1) @ g * (2 * math.pi)
        return torch.cat([c.sin(), c.cos()], -1)

    def _prompt_fourier(self, coords: torch.Tensor) -> torch.Tensor:
        g = self._t("prompt_encoder.shared_embedding.positional_embedding").float()
        c = (2 * coords.float() - 1) @ g * (2 * math.pi)
        return torch.cat([c.sin(), c.cos()], -1)

    def _embed_prompts(self, points, labels, boxes):
        """points [B, P, N, 2] pixels of the model's input, labels [B, P, N] (1 foreground, 0 background,
        -1 not a point, -10 padding), boxes [B, P, 4] -> sparse tokens [B, P, T, hidden] fp32."""
        size = float(self.cfg.prompt_image_size)
        pe = self._t("prompt_encoder.point_embed.weight").float()
        nap = self._t("prompt_encoder.not_a_point_embed.weight").float()
        out = None
        if points is not None:
            pts, lab = points.float().to(self.device) + 0.5, labels.to(self.device)
            if boxes is None:                                          # one padding point closes the point list
                pts = F.pad(pts, (0, 0, 0, 1))
                lab = F.pad(lab, (0, 1), value=-1)
            e = self._prompt_fourier(pts / size)
            e = torch.where(lab[..., None] == -1, nap.expand_as(e), e)
            e = torch.where(lab[..., None] != -10, e, torch.zeros_like(e))
            out = e + pe[lab.clamp(min=0)] * (lab >= 0)[..., None]
        if boxes is not None:
            c = (boxes.float().to(self.device) + 0.5).view(*boxes.shape[:2], 2, 2)
            c = F.pad(c, (0, 0, 0, 1))
            e = self._prompt_fourier(c / size)
            e[:, :, 0] += pe[2]
            e[:, :, 1] += pe[3]
            e[:, :, 2] = nap.expand_as(e[:, :, 2])
            out = e if out is None else torch.cat([out, e], 2)
        return out

    def _dense_prompt(self, masks, batch: int, h: int, w: int):
        if masks is None:
            return self._t("prompt_encoder.no_mask_embed.weight").reshape(1, -1, 1, 1).expand(batch, -1, h, w)
        cfg = self.cfg
        size = 4 * cfg.prompt_image_size // cfg.prompt_patch
        m = masks.float().to(self.device)
        if m.shape[-2:] != (size, size):
            m = F.interpolate(m, size=(size, size), mode="bilinear", align_corners=False, antialias=True)
        p = "prompt_encoder.mask_embed"
        x = F.gelu(self._ln2d(self._conv(m.to(self.dtype), p + ".conv1", 2), p + ".layer_norm1", cfg.prompt_eps))
        x = F.gelu(self._ln2d(self._conv(x, p + ".conv2", 2), p + ".layer_norm2", cfg.prompt_eps))
        return self._conv(x, p + ".conv3")

    # ------------------------------------------------------------------------------ mask decoder
    def _attn(self, q, k, v, p: str, heads: int):
        b = q.shape[0]
        split = lambda t, n: self._lin(t, f"{p}.{n}_proj").view(b, t.shape[1], heads, -1).transpose(1, 2)
        o = F.scaled_dot_product_attention(split(q, "q"), split(k, "k"), split(v, "v")).transpose(1, 2).reshape(b, q.shape[1], -1)
        return self._lin(o, p + ".o_proj")

    def _two_way(self, tokens, image, image_pos):
        """tokens [N, T, C], image [N, HW, C], image_pos [N, HW, C]."""
        cfg = self.cfg
        heads = cfg.decoder_heads
        ln = lambda x, p: self._ln(x, p, 1e-5)
        q, k = tokens, image
        for i in range(cfg.decoder_layers):
            p = f"mask_decoder.transformer.layers.{i}"
            if i == 0:
                q = self._attn(q, q, q, p + ".self_attn", heads)
            else:
                qq = q + tokens
                q = q + self._attn(qq, qq, q, p + ".self_attn", heads)
            q = ln(q, p + ".layer_norm1")
            q = ln(q + self._attn(q + tokens, k + image_pos, k, p + ".cross_attn_token_to_image", heads), p + ".layer_norm2")
            q = ln(q + self._ffn(q, p + ".mlp", cfg.decoder_layers), p + ".layer_norm3")
            k = ln(k + self._attn(k + image_pos, q + tokens, q, p + ".cross_attn_image_to_token", heads), p + ".layer_norm4")
        p = "mask_decoder.transformer"
        q = ln(q + self._attn(q + tokens, k + image_pos, k, p + ".final_attn_token_to_image", heads), p + ".layer_norm_final_attn")
        return q, k

    @torch.no_grad()
    def predict(self, maps: list, points=None, labels=None, boxes=None, masks=None, multimask: bool = True):
        """``maps`` from :meth:`image_embeddings`. Returns (mask logits [B, P, M, 4h, 4w] fp32 at a quarter of the
        input resolution, predicted IoU [B, P, M], object-score logits [B, P, 1]); M = 3 with ``multimask``,
        else 1 (the single-mask token, or the best of the three when that one is unstable)."""
        cfg = self.cfg
        fine, mid, coarse = maps
        b, c, h, w = coarse.shape
        if points is None and boxes is None:
            points = torch.zeros(b, 1, 1, 2)
            labels = -torch.ones(b, 1, 1, dtype=torch.int64)
        if points is not None and labels is None:
            labels = torch.ones(points.shape[:3], dtype=torch.int64)
        sparse = self._embed_prompts(points, labels, boxes).to(self.dtype)           # [B, P, T, C]
        pnum = sparse.shape[1]
        out_tokens = torch.cat([self._t("mask_decoder.obj_score_token.weight"), self._t("mask_decoder.iou_token.weight"),
                                self._t("mask_decoder.mask_tokens.weight")], 0)
        n_mask = cfg.num_multimask_outputs + 1
        tokens = torch.cat([out_tokens[None, None].expand(b, pnum, -1, -1), sparse], 2).reshape(b * pnum, -1, c)
        # position code of the coarse grid: cell centres on [0, 1]
        ys = (torch.arange(h, dtype=torch.float32) + 0.5) / h
        xs = (torch.arange(w, dtype=torch.float32) + 0.5) / w
        grid = torch.stack([xs[None, :].expand(h, w), ys[:, None].expand(h, w)], -1).to(self.device)
        pos = self._fourier(grid).reshape(1, h * w, c).to(self.dtype).expand(b * pnum, -1, -1)
        image = (coarse + self._dense_prompt(masks, b, h, w)).flatten(2).transpose(1, 2).repeat_interleave(pnum, 0)
        q, k = self._two_way(tokens, image, pos)
        iou_tok, mask_toks = q[:, 1], q[:, 2:2 + n_mask]
        img = k.transpose(1, 2).reshape(b * pnum, c, h, w)
        up = F.conv_transpose2d(img, self._t("mask_decoder.upscale_conv1.weight"), self._t("mask_decoder.upscale_conv1.bias"), stride=2)
        up = F.gelu(self._ln2d(up + mid.repeat_interleave(pnum, 0), "mask_decoder.upscale_layer_norm"))
        up = F.conv_transpose2d(up, self._t("mask_decoder.upscale_conv2.weight"), self._t("mask_decoder.upscale_conv2.bias"), stride=2)
        up = F.gelu(up + fine.repeat_interleave(pnum, 0))
        hyper = torch.stack([self._ffn(mask_toks[:, i], f"mask_decoder.output_hypernetworks_mlps.{i}", 3) for i in range(n_mask)], 1)
        hh, ww = up.shape[-2:]
        logits = (hyper.float() @ up.flatten(2).float()).reshape(b, pnum, n_mask, hh, ww)
        iou = self._ffn(iou_tok, "mask_decoder.iou_prediction_head", cfg.iou_head_depth, sigmoid=True).float().reshape(b, pnum, n_mask)
        obj = self._ffn(q[:, 0], "mask_decoder.pred_obj_score_head", 3).float().reshape(b, pnum, 1)
        if multimask:
            return logits[:, :, 1:], iou[:, :, 1:], obj
        if not cfg.dynamic_multimask:
            return logits[:, :, :1], iou[:, :, :1], obj
        # single mask: keep token 0 unless it is unstable, then the best of the other three
        multi, multi_iou = logits[:, :, 1:], iou[:, :, 1:]
        best = multi_iou.argmax(-1)
        pick = best[..., None, None, None].expand(-1, -1, 1, hh, ww)
        best_mask, best_iou = multi.gather(2, pick), multi_iou.gather(2, best[..., None])
        single = logits[:, :, :1]
        flat = single.flatten(-2)
        inner, outer = (flat > cfg.stability_delta).sum(-1).float(), (flat > -cfg.stability_delta).sum(-1).float()
        stable = torch.where(outer > 0, inner / outer, torch.ones_like(outer)) >= cfg.stability_thresh
        return (torch.where(stable[..., None, None], single, best_mask), torch.where(stable, iou[:, :, :1], best_iou), obj)

    @torch.no_grad()
    def segment(self, pixels: torch.Tensor, points=None, labels=None, boxes=None, multimask: bool = True):
        return self.predict(self.image_embeddings(pixels), points, labels, boxes, None, multimask)
