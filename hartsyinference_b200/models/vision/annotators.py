"""Control-image annotators: pictures that condition a ControlNet, made from another picture.

* :func:`canny` - edges: 5 x 5 Gaussian, Sobel gradients, non-maximum suppression along the gradient
  direction quantised to four axes, double threshold, hysteresis (weak pixels survive when chained
  to a strong one). Thresholds are on the 0-255 gradient scale, as in the classic detector.
* :func:`render_pose` - OpenPose-style skeleton picture from body keypoints (the 17 COCO points of
  the pose models here; a neck point is added midway between the shoulders): coloured limbs as
  thick segments and joints as discs on black.
* :func:`depth_control` - a depth map as a grey picture, near = bright, normalised per picture.
* :func:`label_palette` - a label map as a colour picture (a fixed colour per class index).
* :func:`pixelate` / :func:`tile_blur` - the tile / blur hints.

All functions take and return CPU or device tensors and are written with batched tensor operations
(no Python loop over pixels), so they run on the device when given device tensors.
Reference: src/HartsyInference.Vision/ (annotators, OpenPosePreprocessor, OpenPoseRenderer).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F

# the 18-point layout skeletons are drawn in: nose, neck, r-shoulder, r-elbow, r-wrist, l-shoulder, l-elbow, l-wrist,
# r-hip, r-knee, r-ankle, l-hip, l-knee, l-ankle, r-eye, l-eye, r-ear, l-ear
COCO17_TO_BODY18 = (0, -1, 6, 8, 10, 5, 7, 9, 12, 14, 16, 11, 13, 15, 2, 1, 4, 3)
LIMBS = ((1, 2), (1, 5), (2, 3), (3, 4), (5, 6), (6, 7), (1, 8), (8, 9), (9, 10), (1, 11), (11, 12), (12, 13), (1, 0), (0, 14),
         (14, 16), (0, 15), (15, 17))
COLOURS = ((255, 0, 0), (255, 85, 0), (255, 170, 0), (255, 255, 0), (170, 255, 0), (85, 255, 0), (0, 255, 0), (0, 255, 85),
           (0, 255, 170), (0, 255, 255), (0, 170, 255), (0, 85, 255), (0, 0, 255), (85, 0, 255), (170, 0, 255), (255, 0, 255),
           (255, 0, 170), (255, 0, 85))


def _grey(image: torch.Tensor) -> torch.Tensor:
    """[3, H, W] or [H, W] in [0, 1] -> [H, W] on the 0-255 scale."""
    x = image.float()
    if x.dim() == 3:
        x = 0.299 * x[0] + 0.587 * x[1] + 0.114 * x[2]
    return x * 255.0


@torch.no_grad()
def canny(image: torch.Tensor, low: float = 100.0, high: float = 200.0) -> torch.Tensor:
    """-> edge map [H, W] bool."""
    g = _grey(image)[None, None]
    k = torch.tensor([1.0, 4.0, 6.0, 4.0, 1.0], device=g.device) / 16.0
    g = F.conv2d(F.pad(g, (2, 2, 2, 2), mode="reflect"), (k[:, None] * k[None, :])[None, None])
    sx = torch.tensor([[-1.0, 0.0, 1.0], [-2.0, 0.0, 2.0], [-1.0, 0.0, 1.0]], device=g.device)
    p = F.pad(g, (1, 1, 1, 1), mode="replicate")
    gx, gy = F.conv2d(p, sx[None, None])[0, 0], F.conv2d(p, sx.t()[None, None])[0, 0]
    mag = torch.hypot(gx, gy)
    # direction quantised to 0, 45, 90, 135 degrees; compare with the two neighbours along it
    ang = (torch.rad2deg(torch.atan2(gy, gx)) + 180.0) % 180.0
    sector = (((ang + 22.5) // 45.0) % 4).long()
    mp = F.pad(mag[None, None], (1, 1, 1, 1))[0, 0]
    h, w = mag.shape
    nb = lambda dy, dx: mp[1 + dy:1 + dy + h, 1 + dx:1 + dx + w]
    pairs = ((nb(0, 1), nb(0, -1)), (nb(1, 1), nb(-1, -1)), (nb(1, 0), nb(-1, 0)), (nb(1, -1), nb(-1, 1)))
    keep = torch.zeros_like(mag, dtype=torch.bool)
    for s, (a, b) in enumerate(pairs):
        keep |= (sector == s) & (mag >= a) & (mag >= b)
    thin = mag * keep
    strong, weak = thin >= high, thin >= low
    edges = strong.clone()
    while True:                                        # hysteresis: grow the strong set through weak pixels
        grown = (F.max_pool2d(edges[None, None].float(), 3, 1, 1)[0, 0] > 0) & weak
        if torch.equal(grown, edges):
            return edges
        edges = grown


def body18(keypoints: torch.Tensor, min_score: float = 0.3) -> torch.Tensor:
    """COCO keypoints [17, 3] (x, y, visibility) -> [18, 3] in the drawing layout; a neck from the shoulders."""
    k = keypoints.float()
    out = torch.zeros(18, 3)
    for i, src in enumerate(COCO17_TO_BODY18):
        if src >= 0:
            out[i] = k[src]
    ls, rs = k[5], k[6]
    out[1] = torch.stack([(ls[0] + rs[0]) / 2, (ls[1] + rs[1]) / 2, torch.minimum(ls[2], rs[2])])
    out[:, 2] = (out[:, 2] >= min_score).float()
    return out


@torch.no_grad()
def render_pose(people: list, height: int, width: int, thickness: Optional[float] = None, min_score: float = 0.3) -> torch.Tensor:
    """people: COCO keypoint tensors [17, 3] in pixels -> uint8 picture [H, W, 3] of the skeletons on black."""
    canvas = torch.zeros(height, width, 3)
    t = thickness if thickness is not None else max(2.0, min(height, width) / 128.0)
    ys, xs = torch.meshgrid(torch.arange(height, dtype=torch.float32), torch.arange(width, dtype=torch.float32), indexing="ij")
    for kp in people:
        pts = body18(kp, min_score)
        for li, (a, b) in enumerate(LIMBS):
            if pts[a, 2] == 0 or pts[b, 2] == 0:
                continue
            ax, ay, bx, by = pts[a, 0], pts[a, 1], pts[b, 0], pts[b, 1]
            dx, dy = bx - ax, by - ay
            length2 = (dx * dx + dy * dy).clamp_min(1e-6)
            u = (((xs - ax) * dx + (ys - ay) * dy) / length2).clamp(0, 1)
            dist = torch.hypot(xs - (ax + u * dx), ys - (ay + u * dy))
            colour = torch.tensor(COLOURS[li % len(COLOURS)], dtype=torch.float32) * 0.6
            canvas[dist <= t] = colour
        for pi in range(18):
            if pts[pi, 2] == 0:
                continue
            disc = torch.hypot(xs - pts[pi, 0], ys - pts[pi, 1]) <= t * 1.25
            canvas[disc] = torch.tensor(COLOURS[pi % len(COLOURS)], dtype=torch.float32)
    return canvas.round().to(torch.uint8)


def depth_control(depth: torch.Tensor) -> torch.Tensor:
    """relative depth [H, W] (larger = nearer, as Depth Anything writes it) -> uint8 [H, W, 3]."""
    d = depth.float()
    lo, hi = d.min(), d.max()
    g = ((d - lo) / (hi - lo).clamp_min(1e-6) * 255.0).round().to(torch.uint8)
    return g[..., None].expand(-1, -1, 3).contiguous()


def label_palette(labels: torch.Tensor) -> torch.Tensor:
    """label map [H, W] -> uint8 [H, W, 3]; colour of class c: bit-interleaved (the PASCAL colour-map rule)."""
    c = labels.long().clone()
    rgb = torch.zeros(*labels.shape, 3, dtype=torch.long, device=labels.device)
    for j in range(8):
        for ch in range(3):
            rgb[..., ch] |= ((c >> ch) & 1) << (7 - j)
        c >>= 3
    return rgb.to(torch.uint8)


def pixelate(image: torch.Tensor, factor: int = 8) -> torch.Tensor:
    """[3, H, W] -> the picture averaged over ``factor`` x ``factor`` cells, at its own size (tile hint)."""
    h, w = image.shape[-2:]
    small = F.adaptive_avg_pool2d(image[None].float(), (max(1, h // factor), max(1, w // factor)))
    return F.interpolate(small, size=(h, w), mode="nearest")[0]


def tile_blur(image: torch.Tensor, sigma: float = 3.0) -> torch.Tensor:
    """[3, H, W] -> Gaussian blur (blur hint)."""
    r = max(1, int(math.ceil(3 * sigma)))
    x = torch.arange(-r, r + 1, dtype=torch.float32, device=image.device)
    k = torch.exp(-0.5 * (x / sigma) ** 2)
    k = k / k.sum()
    y = F.pad(image[None].float(), (r, r, r, r), mode="reflect")
    y = F.conv2d(y, k.view(1, 1, 1, -1).expand(3, 1, 1, -1), groups=3)
    return F.conv2d(y, k.view(1, 1, -1, 1).expand(3, 1, -1, 1), groups=3)[0]
