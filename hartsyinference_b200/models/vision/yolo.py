"""YOLOv8 object detection (anchor-free, one stage).

Layers are numbered as in the model's definition file (``model.N.*`` tensor names):

* 0-9 backbone: stride-2 3x3 convolutions alternating with C2f blocks (a 1x1 convolution split in two
  halves, a chain of 3x3 bottlenecks on the second half whose every output is kept, all concatenated
  and mixed by a 1x1 convolution), then SPPF (three chained 5x5 max-pools concatenated with their input);
* 10-21 neck: two up-sampling merges with the stride-16 / stride-8 maps, then two stride-2 merges back
  down, a C2f after every concatenation; the outputs of layers 15, 18, 21 are the three scales;
* 22 head: per scale a box branch (two 3x3 convolutions + 1x1 to 4 x 16 distance bins) and a class branch
  (two 3x3 + 1x1 to the classes). A box side is the expectation of the softmax over its 16 bins, measured
  in cells from the cell centre.

Every convolution is followed by BatchNorm (folded into it at load, if the checkpoint still has it)
and SiLU. Sizes n / s / m / l / x scale depth and width.

YOLO11 (``arch="11"``) keeps the plan and changes the blocks: C3k2 (a C2f whose bottlenecks halve their
hidden width, or are themselves two-bottleneck CSP blocks in the deep stages and the larger sizes), a C2PSA
block after SPPF (half the channels pass through position-sensitive self-attention + a two-layer 1x1 FFN),
and a class branch built from depthwise + pointwise pairs; the head is layer 23.

Heads beyond boxes: ``task="segment"`` adds a prototype branch on the stride-8 map (3x3, 2x transposed
convolution, 3x3, 1x1 to 32 prototypes) and 32 mask coefficients per cell, a detection's mask is
sigmoid(coefficients . prototypes) inside its box; ``task="pose"`` adds K x D keypoint values per cell
(x, y decoded as (2 v + cell) x stride, the optional third a sigmoid visibility): body pose has 17
keypoints, face detectors of this family 5 landmarks.

Reference: src/HartsyInference.Vision/Detection/ (YoloModel, YoloV11Model, YoloSegModel, YoloV11PoseModel,
YoloPostProcessor, YoloPosePostProcessor, MaskAssembly, NonMaxSuppression) and FaceDetection/YoloV8FaceModel;
weights are read from a state dict with the original ``model.N.*`` names (safetensors or a plain ``.pt``
state dict).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.nn.functional as F

SCALES = {"n": (1 / 3, 0.25, 1024), "s": (1 / 3, 0.50, 1024), "m": (2 / 3, 0.75, 768), "l": (1.0, 1.0, 512), "x": (1.0, 1.25, 512)}
SCALES_11 = {"n": (0.5, 0.25, 1024), "s": (0.5, 0.50, 1024), "m": (0.5, 1.0, 512), "l": (1.0, 1.0, 512), "x": (1.0, 1.5, 512)}
REG_MAX = 16
PROTOTYPES = 32


@dataclass(frozen=True)
class YoloConfig:
    depth: float = 1 / 3
    width: float = 0.25
    max_channels: int = 1024
    num_classes: int = 80
    arch: str = "v8"                # "v8" or "11"
    task: str = "detect"            # "detect", "segment" or "pose"
    keypoints: int = 0              # pose: points per detection ...
    kpt_dims: int = 3               # ... and values per point (x, y[, visibility])
    csp_inner: bool = False         # YOLO11 m / l / x: every C3k2 holds CSP blocks, not plain bottlenecks

    @property
    def head_layer(self) -> int:
        return 23 if self.arch == "11" else 22

    def ch(self, c: int) -> int:
        return int(math.ceil(min(c, self.max_channels) * self.width / 8) * 8)

    def reps(self, n: int) -> int:
        return max(round(n * self.depth), 1)


def yolo_config(size: str = "n", num_classes: int = 80, arch: str = "v8", task: str = "detect", keypoints: int = 0,
                kpt_dims: int = 3) -> YoloConfig:
    d, w, m = (SCALES_11 if arch == "11" else SCALES)[size]
    if task == "pose" and keypoints == 0:
        keypoints = 17
    return YoloConfig(d, w, m, num_classes, arch, task, keypoints if task == "pose" else 0, kpt_dims,
                      arch == "11" and size in "mlx")


def detect_size(get: Callable) -> YoloConfig:
    """Architecture, size, task and class count from a checkpoint's tensor shapes."""
    w0 = get("model.0.conv.weight")
    if w0 is None:
        raise KeyError("model.0.conv.weight")
    arch = "11" if get("model.10.cv1.conv.weight") is not None else "v8"
    head = 23 if arch == "11" else 22
    first = w0.shape[0]                                   # 64 x width
    top = get("model.7.conv.weight").shape[0]
    nc = get(f"model.{head}.cv3.0.2.weight").shape[0]
    task, kpts, dims = "detect", 0, 3
    if get(f"model.{head}.proto.cv1.conv.weight") is not None:
        task = "segment"
    elif get(f"model.{head}.cv4.0.2.weight") is not None:
        task = "pose"
        nk = get(f"model.{head}.cv4.0.2.weight").shape[0]
        dims = 3 if nk % 3 == 0 else 2
        kpts = nk // dims
    depth_probe = 0
    while get(f"model.2.m.{depth_probe}.cv1.conv.weight") is not None:
        depth_probe += 1
    inner = get("model.2.m.0.cv3.conv.weight") is not None
    for name in "nsmlx":
        cfg = yolo_config(name, nc, arch, task, kpts, dims)
        reps = cfg.reps(3 if arch == "v8" else 2)
        if cfg.ch(64) == first and reps == depth_probe and cfg.ch(1024) == top and (arch == "v8" or cfg.csp_inner == inner):
            return cfg
    raise ValueError(f"unrecognised YOLO size (first width {first}, {depth_probe} blocks in stage 2, top width {top})")


class YoloV8:
    def __init__(self, cfg: YoloConfig, device="cpu", get: Optional[Callable[[str], Optional[torch.Tensor]]] = None, seed: int = 0,
                 dtype: Optional[torch.dtype] = None):
        self.cfg, self.device = cfg, torch.device(device)
        self.dtype = dtype or (torch.bfloat16 if self.device.type == "cuda" else torch.float32)
        self._get, self._g = get, torch.Generator().manual_seed(seed)
        self._w: dict = {}
        self.param_count = 0            # parameters of the unfolded model (convolution + BatchNorm scale / shift)

    @property
    def param_count_total(self) -> int:
        """After one forward: the published parameter count (with the fixed bin-index kernel of the head)."""
        return self.param_count + REG_MAX

    # ------------------------------------------------------------------------------ weights
    def _conv_bn(self, p: str, co: int, ci: int, k: int):
        hit = self._w.get(p)
        if hit is None:
            if self._get is None:
                w = torch.randn(co, ci, k, k, generator=self._g) * (1.0 / (ci * k * k)) ** 0.5
                b = torch.randn(co, generator=self._g) * 0.1
            else:
                w = self._get(p + ".conv.weight").float()
                b = self._get(p + ".conv.bias")
                g = self._get(p + ".bn.weight")
                if g is not None:                          # BatchNorm still separate: fold it (eps 1e-3 in this family)
                    s = g.float() * torch.rsqrt(self._get(p + ".bn.running_var").float() + 1e-3)
                    w = w * s[:, None, None, None]
                    b = self._get(p + ".bn.bias").float() - self._get(p + ".bn.running_mean").float() * s
                else:
                    b = torch.zeros(co) if b is None else b.float()
            assert w.shape == (co, ci, k, k), (p, tuple(w.shape), (co, ci, k, k))
            self.param_count += co * ci * k * k + 2 * co
            hit = (w.to(self.device).to(self.dtype), b.to(self.device).to(self.dtype))
            self._w[p] = hit
        return hit

    def _plain(self, p: str, co: int, ci: int):
        hit = self._w.get(p)
        if hit is None:
            if self._get is None:
                w, b = torch.randn(co, ci, 1, 1, generator=self._g) * (1.0 / ci) ** 0.5, torch.zeros(co)
            else:
                w, b = self._get(p + ".weight").float(), self._get(p + ".bias").float()
            self.param_count += co * ci + co
            hit = (w.reshape(co, ci, 1, 1).to(self.device).to(self.dtype), b.to(self.device).to(self.dtype))
            self._w[p] = hit
        return hit

    def _transposed(self, p: str, c: int):
        hit = self._w.get(p)
        if hit is None:
            if self._get is None:
                w, b = torch.randn(c, c, 2, 2, generator=self._g) * (1.0 / (4 * c)) ** 0.5, torch.zeros(c)
            else:
                w, b = self._get(p + ".weight").float(), self._get(p + ".bias").float()
            self.param_count += w.numel() + c
            hit = (w.to(self.device).to(self.dtype), b.to(self.device).to(self.dtype))
            self._w[p] = hit
        return hit

    # ------------------------------------------------------------------------------ blocks
    def _conv(self, x, p: str, co: int, k: int = 1, s: int = 1, act: bool = True, depthwise: bool = False):
        ci = x.shape[1]
        w, b = self._conv_bn(p, co, 1 if depthwise else ci, k)
        y = F.conv2d(x, w, b, stride=s, padding=k // 2, groups=ci if depthwise else 1)
        return F.silu(y) if act else y

    def _bottleneck(self, x, p: str, c: int, shortcut: bool, e: float):
        h = self._conv(self._conv(x, p + ".cv1", int(c * e), 3), p + ".cv2", c, 3)
        return x + h if shortcut else h

    def _c2f(self, x, p: str, co: int, n: int, shortcut: bool, e: float = 0.5, csp: bool = False):
        """C2f (``csp`` False, full-width bottlenecks) and C3k2 (half-width bottlenecks, or CSP blocks of two)."""
        c = int(co * e)
        y = list(self._conv(x, p + ".cv1", 2 * c).chunk(2, 1))
        for i in range(n):
            q = f"{p}.m.{i}"
            if csp:
                h = c // 2
                t = self._conv(y[-1], q + ".cv1", h)
                for j in range(2):
                    t = self._bottleneck(t, f"{q}.m.{j}", h, shortcut, 1.0)
                y.append(self._conv(torch.cat([t, self._conv(y[-1], q + ".cv2", h)], 1), q + ".cv3", c))
            else:
                y.append(self._bottleneck(y[-1], q, c, shortcut, 1.0 if self.cfg.arch == "v8" else 0.5))
        return self._conv(torch.cat(y, 1), p + ".cv2", co)

    def _sppf(self, x, p: str, co: int):
        y = [self._conv(x, p + ".cv1", x.shape[1] // 2)]
        for _ in range(3):
            y.append(F.max_pool2d(y[-1], 5, 1, 2))
        return self._conv(torch.cat(y, 1), p + ".cv2", co)

    def _c2psa(self, x, p: str, n: int):
        c = x.shape[1] // 2
        a, b = self._conv(x, p + ".cv1", 2 * c).split((c, c), 1)
        heads = max(c // 64, 1)
        hd = c // heads
        kd = hd // 2
        for i in range(n):
            q = f"{p}.m.{i}"
            bs, _, h, w = b.shape
            qkv = self._conv(b, q + ".attn.qkv", c + 2 * kd * heads, act=False).view(bs, heads, 2 * kd + hd, h * w)
            qq, kk, vv = qkv.split([kd, kd, hd], 2)
            att = ((qq.transpose(-2, -1).float() @ kk.float()) * kd ** -0.5).softmax(-1).to(vv.dtype)
            o = (vv @ att.transpose(-2, -1)).reshape(bs, c, h, w)
            o = o + self._conv(vv.reshape(bs, c, h, w), q + ".attn.pe", c, 3, act=False, depthwise=True)
            b = b + self._conv(o, q + ".attn.proj", c, act=False)
            b = b + self._conv(self._conv(b, q + ".ffn.0", 2 * c), q + ".ffn.1", c, act=False)
        return self._conv(torch.cat([a, b], 1), p + ".cv2", x.shape[1])

    @torch.no_grad()
    def features(self, x: torch.Tensor) -> list:
        c, r = self.cfg.ch, self.cfg.reps
        m = lambda i: f"model.{i}"
        up = lambda t: F.interpolate(t, scale_factor=2.0, mode="nearest")
        if self.cfg.arch == "11":
            inner = self.cfg.csp_inner
            n = r(2)
            x = self._conv(x, m(0), c(64), 3, 2)
            x = self._conv(x, m(1), c(128), 3, 2)
            x = self._c2f(x, m(2), c(256), n, True, 0.25, inner)
            x = self._conv(x, m(3), c(256), 3, 2)
            p3 = self._c2f(x, m(4), c(512), n, True, 0.25, inner)
            x = self._conv(p3, m(5), c(512), 3, 2)
            p4 = self._c2f(x, m(6), c(512), n, True, 0.5, True)
            x = self._conv(p4, m(7), c(1024), 3, 2)
            x = self._c2f(x, m(8), c(1024), n, True, 0.5, True)
            p5 = self._c2psa(self._sppf(x, m(9), c(1024)), m(10), n)
            n4 = self._c2f(torch.cat([up(p5), p4], 1), m(13), c(512), n, True, 0.5, inner)
            n3 = self._c2f(torch.cat([up(n4), p3], 1), m(16), c(256), n, True, 0.5, inner)
            d4 = self._c2f(torch.cat([self._conv(n3, m(17), c(256), 3, 2), n4], 1), m(19), c(512), n, True, 0.5, inner)
            d5 = self._c2f(torch.cat([self._conv(d4, m(20), c(512), 3, 2), p5], 1), m(22), c(1024), n, True, 0.5, True)
            return [n3, d4, d5]
        x = self._conv(x, m(0), c(64), 3, 2)
        x = self._conv(x, m(1), c(128), 3, 2)
        x = self._c2f(x, m(2), c(128), r(3), True)
        x = self._conv(x, m(3), c(256), 3, 2)
        p3 = self._c2f(x, m(4), c(256), r(6), True)
        x = self._conv(p3, m(5), c(512), 3, 2)
        p4 = self._c2f(x, m(6), c(512), r(6), True)
        x = self._conv(p4, m(7), c(1024), 3, 2)
        x = self._c2f(x, m(8), c(1024), r(3), True)
        p5 = self._sppf(x, m(9), c(1024))
        n4 = self._c2f(torch.cat([up(p5), p4], 1), m(12), c(512), r(3), False)
        n3 = self._c2f(torch.cat([up(n4), p3], 1), m(15), c(256), r(3), False)
        d4 = self._c2f(torch.cat([self._conv(n3, m(16), c(256), 3, 2), n4], 1), m(18), c(512), r(3), False)
        d5 = self._c2f(torch.cat([self._conv(d4, m(19), c(512), 3, 2), p5], 1), m(21), c(1024), r(3), False)
        return [n3, d4, d5]

    def _branch(self, f, p: str, width: int, out: int, light: bool = False):
        """Two 3x3 stages and a plain 1x1: the shape of every head branch. ``light``: each 3x3 is a depthwise 3x3
        followed by a pointwise 1x1 (the class branch of YOLO11)."""
        t = f
        for j in range(2):
            if light:
                t = self._conv(self._conv(t, f"{p}.{j}.0", t.shape[1], 3, depthwise=True), f"{p}.{j}.1", width)
            else:
                t = self._conv(t, f"{p}.{j}", width, 3)
        return F.conv2d(t, *self._plain(f"{p}.2", out, width)).float()

    @torch.no_grad()
    def forward_all(self, pixels: torch.Tensor) -> dict:
        """pixels [B, 3, H, W] in [0, 1] (H, W multiples of 32) -> dict of fp32 tensors over all A cells of the
        three scales: ``boxes`` [B, A, 4] (x0, y0, x1, y1 in input pixels), ``scores`` [B, A, classes]; with a
        segment head ``coefficients`` [B, A, 32] and ``prototypes`` [B, 32, H/4, W/4]; with a pose head
        ``keypoints`` [B, A, K, D] (x, y in input pixels, visibility as a probability)."""
        cfg = self.cfg
        feats = self.features(pixels.to(self.device).to(self.dtype))
        head = f"model.{cfg.head_layer}"
        c0 = feats[0].shape[1]
        c2 = max(16, c0 // 4, 4 * REG_MAX)
        c3 = max(c0, min(cfg.num_classes, 100))
        nk = cfg.keypoints * cfg.kpt_dims
        boxes, scores, extra = [], [], []
        for i, f in enumerate(feats):
            b, _, h, w = f.shape
            stride = pixels.shape[-1] / w
            dist = self._branch(f, f"{head}.cv2.{i}", c2, 4 * REG_MAX)
            cls = self._branch(f, f"{head}.cv3.{i}", c3, cfg.num_classes, light=cfg.arch == "11")
            d = (dist.view(b, 4, REG_MAX, h * w).softmax(2) * torch.arange(REG_MAX, device=f.device).view(1, 1, -1, 1)).sum(2)
            ys, xs = torch.meshgrid(torch.arange(h, device=f.device) + 0.5, torch.arange(w, device=f.device) + 0.5, indexing="ij")
            cx, cy = xs.reshape(1, -1), ys.reshape(1, -1)
            boxes.append(torch.stack([cx - d[:, 0], cy - d[:, 1], cx + d[:, 2], cy + d[:, 3]], -1) * stride)
            scores.append(cls.view(b, cfg.num_classes, h * w).transpose(1, 2).sigmoid())
            if cfg.task == "segment":
                co = self._branch(f, f"{head}.cv4.{i}", max(c0 // 4, PROTOTYPES), PROTOTYPES)
                extra.append(co.view(b, PROTOTYPES, h * w).transpose(1, 2))
            elif cfg.task == "pose":
                k = self._branch(f, f"{head}.cv4.{i}", max(c0 // 4, nk), nk).view(b, cfg.keypoints, cfg.kpt_dims, h * w)
                kx = (k[:, :, 0] * 2.0 + (cx - 0.5)[:, None]) * stride
                ky = (k[:, :, 1] * 2.0 + (cy - 0.5)[:, None]) * stride
                parts = [kx, ky] + ([k[:, :, 2].sigmoid()] if cfg.kpt_dims == 3 else [])
                extra.append(torch.stack(parts, 2).permute(0, 3, 1, 2))
        out = {"boxes": torch.cat(boxes, 1), "scores": torch.cat(scores, 1)}
        if cfg.task == "segment":
            npr = cfg.ch(256)
            t = self._conv(feats[0], f"{head}.proto.cv1", npr, 3)
            t = F.conv_transpose2d(t, *self._transposed(f"{head}.proto.upsample", npr), stride=2)
            t = self._conv(self._conv(t, f"{head}.proto.cv2", npr, 3), f"{head}.proto.cv3", PROTOTYPES)
            out["coefficients"], out["prototypes"] = torch.cat(extra, 1), t.float()
        elif cfg.task == "pose":
            out["keypoints"] = torch.cat(extra, 1)
        return out

    def forward(self, pixels: torch.Tensor):
        """(boxes [B, A, 4], class probabilities [B, A, classes]) of :meth:`forward_all`."""
        out = self.forward_all(pixels)
        return out["boxes"], out["scores"]

    @torch.no_grad()
    def detect(self, pixels: torch.Tensor, threshold: float = 0.25, iou: float = 0.7, max_det: int = 300,
               full: bool = False) -> list:
        """Per image a list of (class id, score, (x0, y0, x1, y1) in input pixels), best first, after
        class-wise non-maximum suppression. ``full``: each entry is a dict that also carries ``mask``
        (bool [H, W] at input resolution, segment head) or ``keypoints`` ([K, D], pose head)."""
        from ...engine.vision_service import nms
        raw = self.forward_all(pixels)
        hh, ww = pixels.shape[-2:]
        out = []
        for n, (bx, sc) in enumerate(zip(raw["boxes"].cpu(), raw["scores"].cpu())):
            conf, cls = sc.max(-1)
            sel = (conf >= threshold).nonzero().flatten()
            sel = sel[conf[sel].argsort(descending=True)[:3000]]
            shifted = bx[sel] + cls[sel, None].float() * 7680.0        # classes never suppress each other
            kept = [int(sel[i]) for i in nms(shifted, conf[sel], iou)[:max_det]]
            found = []
            for i in kept:
                box = tuple(bx[i].tolist())
                if not full:
                    found.append((int(cls[i]), float(conf[i]), box))
                    continue
                d = {"label": int(cls[i]), "score": float(conf[i]), "box": box}
                if "keypoints" in raw:
                    d["keypoints"] = raw["keypoints"][n, i].cpu()
                if "prototypes" in raw:
                    proto = raw["prototypes"][n]
                    m = (raw["coefficients"][n, i] @ proto.flatten(1)).view(1, 1, *proto.shape[-2:]).sigmoid()
                    m = F.interpolate(m, size=(hh, ww), mode="bilinear", align_corners=False)[0, 0].cpu() > 0.5
                    inside = torch.zeros_like(m)
                    x0, y0, x1, y1 = (int(max(v, 0)) for v in (box[0], box[1], box[2] + 1, box[3] + 1))
                    inside[y0:y1, x0:x1] = True
                    d["mask"] = m & inside
                found.append(d)
            out.append(found)
        return out
