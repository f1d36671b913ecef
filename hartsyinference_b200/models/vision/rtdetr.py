"""RT-DETR closed-set object detection (ResNet-vd backbone, hybrid encoder, deformable decoder).

Pipeline of one image (all batch-norms folded into their convolutions at load):

* backbone: three-convolution stem + max-pool, four stages of basic or bottleneck residual blocks
  whose down-sampling shortcuts average-pool first ("vd"); the last three stages feed the neck;
* hybrid encoder: 1x1 projections to one width, a transformer layer with 2-d sine / cosine
  positions on the coarsest map only, then a top-down and a bottom-up pass of cross-stage-partial
  blocks built from re-parameterisable 3x3 + 1x1 convolution pairs;
* query selection: every location of the three maps proposes a class score and a box (anchor grid +
  regressed offset); the ``num_queries`` best-scoring locations become the decoder's queries and
  reference boxes;
* decoder: self-attention over the queries, multi-scale deformable attention into the three maps
  (``ops.msda``: softmax, sampling locations, bilinear gathers and weighted sum in one kernel on the
  device), feed-forward; each layer refines the reference boxes, the last layer's class head scores
  them.

Reference: src/HartsyInference.Vision/Detection/ (closed-set detectors behind the vision service's
detect operation; its deformable-attention kernel is src/HartsyInference.Cuda/Kernels/vision/msda.cu).
Tensor names follow Hugging Face ``RTDetrForObjectDetection``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, Optional

import torch
import torch.nn.functional as F

from ... import ops

_ACT = {"relu": F.relu, "silu": F.silu, "gelu": F.gelu, None: lambda x: x}


@dataclass
class RtDetrConfig:
    # backbone
    embedding_size: int = 64
    hidden_sizes: tuple = (256, 512, 1024, 2048)
    depths: tuple = (3, 4, 6, 3)
    layer_type: str = "bottleneck"
    backbone_act: str = "relu"
    downsample_in_first_stage: bool = False
    downsample_in_bottleneck: bool = False
    out_stages: tuple = (1, 2, 3)               # indices into the four stages
    # hybrid encoder
    encoder_hidden_dim: int = 256
    feat_strides: tuple = (8, 16, 32)
    encoder_layers: int = 1
    encoder_ffn_dim: int = 1024
    encoder_heads: int = 8
    encode_proj_layers: tuple = (2,)
    pe_temperature: float = 10000.0
    hidden_expansion: float = 1.0
    activation: str = "silu"
    encoder_activation: str = "gelu"
    normalize_before: bool = False
    eval_size: Optional[tuple] = None
    # decoder
    d_model: int = 256
    num_queries: int = 300
    decoder_ffn_dim: int = 1024
    num_feature_levels: int = 3
    decoder_points: int = 4
    decoder_layers: int = 6
    decoder_heads: int = 8
    decoder_activation: str = "relu"
    layer_norm_eps: float = 1e-5
    batch_norm_eps: float = 1e-5
    num_labels: int = 80
    learn_initial_query: bool = False
    image_size: int = 640
    id2label: dict = field(default_factory=dict)


def rtdetr_from_hf(d: dict) -> RtDetrConfig:
    b = d.get("backbone_config") or {}
    stages = b.get("out_indices") or [2, 3, 4]
    return RtDetrConfig(
        embedding_size=b.get("embedding_size", 64), hidden_sizes=tuple(b.get("hidden_sizes", (256, 512, 1024, 2048))),
        depths=tuple(b.get("depths", (3, 4, 6, 3))), layer_type=b.get("layer_type", "bottleneck"),
        backbone_act=b.get("hidden_act", "relu"), downsample_in_first_stage=bool(b.get("downsample_in_first_stage", False)),
        downsample_in_bottleneck=bool(b.get("downsample_in_bottleneck", False)), out_stages=tuple(int(i) - 1 for i in stages),
        encoder_hidden_dim=d.get("encoder_hidden_dim", 256), feat_strides=tuple(d.get("feat_strides", (8, 16, 32))),
        encoder_layers=d.get("encoder_layers", 1), encoder_ffn_dim=d.get("encoder_ffn_dim", 1024),
        encoder_heads=d.get("encoder_attention_heads", 8), encode_proj_layers=tuple(d.get("encode_proj_layers", (2,))),
        pe_temperature=float(d.get("positional_encoding_temperature", 10000)), hidden_expansion=float(d.get("hidden_expansion", 1.0)),
        activation=d.get("activation_function", "silu"), encoder_activation=d.get("encoder_activation_function", "gelu"),
        normalize_before=bool(d.get("normalize_before", False)),
        eval_size=tuple(d["eval_size"]) if d.get("eval_size") else None, d_model=d.get("d_model", 256),
        num_queries=d.get("num_queries", 300), decoder_ffn_dim=d.get("decoder_ffn_dim", 1024),
        num_feature_levels=d.get("num_feature_levels", 3), decoder_points=d.get("decoder_n_points", 4),
        decoder_layers=d.get("decoder_layers", 6), decoder_heads=d.get("decoder_attention_heads", 8),
        decoder_activation=d.get("decoder_activation_function", "relu"), layer_norm_eps=float(d.get("layer_norm_eps", 1e-5)),
        batch_norm_eps=float(d.get("batch_norm_eps", 1e-5)),
        num_labels=len(d["id2label"]) if d.get("id2label") else d.get("num_labels", 80),
        learn_initial_query=bool(d.get("learn_initial_query", False)),
        image_size=int((d.get("anchor_image_size") or [640, 640])[0]),
        id2label={int(k): v for k, v in (d.get("id2label") or {}).items()})


class RtDetr:
    """``get(name)`` returns checkpoint tensors by their Hugging Face names. Inference only."""

    def __init__(self, cfg: RtDetrConfig, device="cpu", get: Optional[Callable[[str], Optional[torch.Tensor]]] = None,
                 dtype: Optional[torch.dtype] = None):
        self.cfg, self.device = cfg, torch.device(device)
        self.dtype = dtype or (torch.bfloat16 if self.device.type == "cuda" else torch.float32)
        if get is None:
            raise ValueError("RT-DETR needs a checkpoint")
        self._get = get
        self._w: dict = {}

    # ------------------------------------------------------------------------------ weights
    def _t(self, name: str, optional: bool = False) -> Optional[torch.Tensor]:
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

    def _has(self, name: str) -> bool:
        return name in self._w or self._get(name) is not None

    def _conv_bn(self, conv: str, bn: str, eps: float):
        """Convolution weight with its (frozen) batch-norm folded in: (weight, bias)."""
        key = conv + "|" + bn
        hit = self._w.get(key)
        if hit is None:
            w = self._get(conv + ".weight").float()
            g, b = self._get(bn + ".weight").float(), self._get(bn + ".bias").float()
            mean, var = self._get(bn + ".running_mean").float(), self._get(bn + ".running_var").float()
            s = g * torch.rsqrt(var + eps)
            hit = ((w * s[:, None, None, None]).to(self.device).to(self.dtype), (b - mean * s).to(self.device).to(self.dtype))
            self._w[key] = hit
        return hit

    def _cba(self, x, conv: str, bn: str, eps: float, stride: int = 1, act: Optional[str] = None):
        w, b = self._conv_bn(conv, bn, eps)
        return _ACT[act](F.conv2d(x, w, b, stride=stride, padding=w.shape[-1] // 2))

    def _linear(self, x, prefix: str):
        return F.linear(x, self._t(prefix + ".weight"), self._t(prefix + ".bias", optional=True))

    def _ln(self, x, prefix: str):
        return F.layer_norm(x, (x.shape[-1],), self._t(prefix + ".weight"), self._t(prefix + ".bias"), self.cfg.layer_norm_eps)

    def _mlp_head(self, x, prefix: str, layers: int):
        for i in range(layers):
            x = self._linear(x, f"{prefix}.layers.{i}")
            if i < layers - 1:
                x = F.relu(x)
        return x

    # ------------------------------------------------------------------------------ backbone
    def _res_block(self, x, p: str, stride: int):
        cfg = self.cfg
        eps = 1e-5
        unit = lambda h, i, s, a: self._cba(h, f"{p}.layer.{i}.convolution", f"{p}.layer.{i}.normalization", eps, s, a)
        if cfg.layer_type == "bottleneck":
            h = unit(x, 0, stride if cfg.downsample_in_bottleneck else 1, cfg.backbone_act)
            h = unit(h, 1, 1 if cfg.downsample_in_bottleneck else stride, cfg.backbone_act)
            h = unit(h, 2, 1, None)
        else:
            h = unit(x, 0, stride, cfg.backbone_act)
            h = unit(h, 1, 1, None)
        if self._has(f"{p}.shortcut.1.convolution.weight"):          # average-pool, then a 1x1 projection
            r = F.avg_pool2d(x, 2, 2, 0, ceil_mode=True)
            r = self._cba(r, f"{p}.shortcut.1.convolution", f"{p}.shortcut.1.normalization", eps)
        elif self._has(f"{p}.shortcut.convolution.weight"):
            r = self._cba(x, f"{p}.shortcut.convolution", f"{p}.shortcut.normalization", eps, stride)
        else:
            r = F.avg_pool2d(x, 2, 2, 0, ceil_mode=True) if (stride == 2 and cfg.layer_type == "bottleneck") else x
        return _ACT[cfg.backbone_act](h + r)

    def backbone(self, x: torch.Tensor) -> list:
        cfg = self.cfg
        p = "model.backbone.model."
        for i, s in enumerate((2, 1, 1)):
            x = self._cba(x, f"{p}embedder.embedder.{i}.convolution", f"{p}embedder.embedder.{i}.normalization", 1e-5, s, cfg.backbone_act)
        x = F.max_pool2d(x, 3, 2, 1)
        feats = []
        for si, depth in enumerate(cfg.depths):
            stride = (2 if cfg.downsample_in_first_stage else 1) if si == 0 else 2
            for li in range(depth):
                x = self._res_block(x, f"{p}encoder.stages.{si}.layers.{li}", stride if li == 0 else 1)
            if si in cfg.out_stages:
                feats.append(x)
        return feats

    # ------------------------------------------------------------------------------ hybrid encoder
    def _attention(self, x, pos, prefix: str, heads: int):
        """x [B, T, C]; positions are added to queries and keys only."""
        b, t, c = x.shape
        qk = x if pos is None else x + pos
        shape = (b, t, heads, c // heads)
        q = self._linear(qk, prefix + ".q_proj").view(shape).transpose(1, 2)
        k = self._linear(qk, prefix + ".k_proj").view(shape).transpose(1, 2)
        v = self._linear(x, prefix + ".v_proj").view(shape).transpose(1, 2)
        o = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(b, t, c)
        return self._linear(o, prefix + ".o_proj")

    def _sincos_2d(self, h: int, w: int, dim: int) -> torch.Tensor:
        gy, gx = torch.meshgrid(torch.arange(h, dtype=torch.float32), torch.arange(w, dtype=torch.float32), indexing="ij")
        omega = 1.0 / (self.cfg.pe_temperature ** (torch.arange(dim // 4, dtype=torch.float32) / (dim // 4)))
        oy, ox = gy.reshape(-1, 1) * omega[None], gx.reshape(-1, 1) * omega[None]
        return torch.cat([oy.sin(), oy.cos(), ox.sin(), ox.cos()], 1)[None].to(self.device).to(self.dtype)

    def _aifi(self, x, i: int):
        cfg = self.cfg
        b, c, h, w = x.shape
        t = x.flatten(2).permute(0, 2, 1)
        pos = self._sincos_2d(h, w, c) if cfg.eval_size is None else None
        for li in range(cfg.encoder_layers):
            p = f"model.encoder.aifi.{i}.layers.{li}"
            r = t
            y = self._ln(t, p + ".self_attn_layer_norm") if cfg.normalize_before else t
            t = r + self._attention(y, pos, p + ".self_attn", cfg.encoder_heads)
            if not cfg.normalize_before:
                t = self._ln(t, p + ".self_attn_layer_norm")
            r = t
            y = self._ln(t, p + ".final_layer_norm") if cfg.normalize_before else t
            t = r + self._linear(_ACT[cfg.encoder_activation](self._linear(y, p + ".mlp.fc1")), p + ".mlp.fc2")
            if not cfg.normalize_before:
                t = self._ln(t, p + ".final_layer_norm")
        return t.permute(0, 2, 1).reshape(b, c, h, w).contiguous()

    def _csp(self, x, p: str):
        cfg, eps = self.cfg, self.cfg.batch_norm_eps
        a = self._cba(x, p + ".conv1.conv", p + ".conv1.norm", eps, 1, cfg.activation)
        for i in range(3):
            q = f"{p}.bottlenecks.{i}"
            a = _ACT[cfg.activation](self._cba(a, q + ".conv1.conv", q + ".conv1.norm", eps) +
                                     self._cba(a, q + ".conv2.conv", q + ".conv2.norm", eps))
        y = a + self._cba(x, p + ".conv2.conv", p + ".conv2.norm", eps, 1, cfg.activation)
        if self._has(p + ".conv3.conv.weight"):
            y = self._cba(y, p + ".conv3.conv", p + ".conv3.norm", eps, 1, cfg.activation)
        return y

    def encoder(self, feats: list) -> list:
        cfg, eps = self.cfg, self.cfg.batch_norm_eps
        maps = [self._cba(f, f"model.encoder_input_proj.{i}.0", f"model.encoder_input_proj.{i}.1", 1e-5) for i, f in enumerate(feats)]
        if cfg.encoder_layers > 0:
            for i, at in enumerate(cfg.encode_proj_layers):
                maps[at] = self._aifi(maps[at], i)
        n = len(maps) - 1
        fpn = [maps[-1]]
        for i in range(n):                                           # top-down
            top = self._cba(fpn[-1], f"model.encoder.lateral_convs.{i}.conv", f"model.encoder.lateral_convs.{i}.norm", eps, 1, cfg.activation)
            fpn[-1] = top
            up = F.interpolate(top, scale_factor=2.0, mode="nearest")
            fpn.append(self._csp(torch.cat([up, maps[n - i - 1]], 1), f"model.encoder.fpn_blocks.{i}"))
        fpn.reverse()
        pan = [fpn[0]]
        for i in range(n):                                           # bottom-up
            down = self._cba(pan[-1], f"model.encoder.downsample_convs.{i}.conv", f"model.encoder.downsample_convs.{i}.norm", eps, 2,
                             cfg.activation)
            pan.append(self._csp(torch.cat([down, fpn[i + 1]], 1), f"model.encoder.pan_blocks.{i}"))
        return pan

    # ------------------------------------------------------------------------------ decoder
    def _anchors(self, shapes: list, grid_size: float = 0.05):
        out = []
        for level, (h, w) in enumerate(shapes):
            gy, gx = torch.meshgrid(torch.arange(h, dtype=torch.float32), torch.arange(w, dtype=torch.float32), indexing="ij")
            xy = torch.stack([(gx + 0.5) / w, (gy + 0.5) / h], -1)
            wh = torch.full_like(xy, grid_size * (2.0 ** level))
            out.append(torch.cat([xy, wh], -1).reshape(-1, 4))
        a = torch.cat(out)[None]
        valid = ((a > 1e-2) & (a < 1 - 1e-2)).all(-1, keepdim=True)
        logit = torch.log(a / (1 - a))
        big = torch.finfo(torch.float32).max
        return torch.where(valid, logit, torch.full_like(logit, big)).to(self.device), valid.to(self.device)

    def _deformable(self, x, pos, memory, shapes, ref, p: str):
        cfg = self.cfg
        b, q, c = x.shape
        heads, lv, pts = cfg.decoder_heads, cfg.num_feature_levels, cfg.decoder_points
        y = x + pos
        value = self._linear(memory, p + ".value_proj").view(b, memory.shape[1], heads, c // heads)
        off = self._linear(y, p + ".sampling_offsets").view(b, q, heads, lv, pts, 2)
        logits = self._linear(y, p + ".attention_weights").view(b, q, heads, lv, pts)
        out = ops.msda(value, shapes, off, logits, ref)
        return self._linear(out.to(x.dtype), p + ".output_proj")

    @torch.no_grad()
    def forward(self, pixels: torch.Tensor):
        """pixels [B, 3, H, W] in [0, 1] (H, W multiples of 32). Returns (class logits [B, Q, labels] fp32,
        boxes [B, Q, 4] fp32 as normalised cx, cy, w, h)."""
        cfg = self.cfg
        x = pixels.to(self.device).to(self.dtype)
        maps = self.encoder(self.backbone(x))
        eps = cfg.batch_norm_eps
        srcs = [self._cba(m, f"model.decoder_input_proj.{i}.0", f"model.decoder_input_proj.{i}.1", eps) for i, m in enumerate(maps)]
        shapes = [tuple(s.shape[-2:]) for s in srcs]
        memory = torch.cat([s.flatten(2).transpose(1, 2) for s in srcs], 1)                 # [B, S, C]
        b = memory.shape[0]
        anchors, valid = self._anchors(shapes)
        out_mem = self._ln(self._linear(memory * valid.to(memory.dtype), "model.enc_output.0"), "model.enc_output.1")
        enc_class = self._linear(out_mem, "model.enc_score_head").float()
        enc_box = self._mlp_head(out_mem, "model.enc_bbox_head", 3).float() + anchors
        top = torch.topk(enc_class.max(-1).values, cfg.num_queries, dim=1).indices          # [B, Q]
        ref_unact = enc_box.gather(1, top[..., None].expand(-1, -1, 4))
        if cfg.learn_initial_query:
            target = self._t("model.weight_embedding.weight")[None].expand(b, -1, -1)
        else:
            target = out_mem.gather(1, top[..., None].expand(-1, -1, out_mem.shape[-1]))
        ref = torch.sigmoid(ref_unact)
        h = target
        logits = None
        for li in range(cfg.decoder_layers):
            p = f"model.decoder.layers.{li}"
            pos = self._mlp_head(ref.to(self.dtype), "model.decoder.query_pos_head", 2)
            h = self._ln(h + self._attention(h, pos, p + ".self_attn", cfg.decoder_heads), p + ".self_attn_layer_norm")
            h = self._ln(h + self._deformable(h, pos, memory, shapes, ref, p + ".encoder_attn"), p + ".encoder_attn_layer_norm")
            f = self._linear(_ACT[cfg.decoder_activation](self._linear(h, p + ".mlp.fc1")), p + ".mlp.fc2")
            h = self._ln(h + f, p + ".final_layer_norm")
            corners = self._mlp_head(h, f"model.decoder.bbox_embed.{li}", 3).float()
            r = ref.clamp(0, 1)
            ref = torch.sigmoid(corners + torch.log(r.clamp(min=1e-5) / (1 - r).clamp(min=1e-5)))
            if li == cfg.decoder_layers - 1:
                logits = self._linear(h, f"model.decoder.class_embed.{li}").float()
        return logits, ref

    @torch.no_grad()
    def detect(self, pixels: torch.Tensor, threshold: float = 0.5) -> list:
        """Per image a list of (label id, score, (cx, cy, w, h) normalised), best first: the
        ``num_queries`` highest sigmoid scores over all (query, class) pairs that pass ``threshold``."""
        logits, boxes = self.forward(pixels)
        out = []
        for lg, bx in zip(logits, boxes):
            scores = torch.sigmoid(lg).flatten()
            top = torch.topk(scores, min(self.cfg.num_queries, scores.numel()))
            found = []
            for s, i in zip(top.values.tolist(), top.indices.tolist()):
                if s < threshold:
                    break
                found.append((i % lg.shape[-1], s, tuple(bx[i // lg.shape[-1]].tolist())))
            out.append(found)
        return out
