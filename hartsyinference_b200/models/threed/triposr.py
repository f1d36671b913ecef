"""TripoSR: feed-forward single-image -> triplane radiance field -> mesh.

A DINO ViT-B/16 turns the (512 x 512, grey-composited) image into 1025 tokens; 3 x 32 x 32 learned
triplane tokens run through 16 transformer blocks (self-attention, cross-attention to the image
tokens, GEGLU feed-forward) inside a residual wrapper with a GroupNorm in front; a transposed
convolution doubles each plane to 64 x 64 with 40 channels; a query point is projected onto the three
planes, the 120 sampled features go through a ten-layer SiLU MLP to (density, rgb). Density is
``exp(raw - 1)``, colour ``sigmoid(raw)``; the mesh is the iso-surface of the density at 25 on a
lattice over [-0.87, 0.87]^3.

On the device the field decode (sampling + MLP) is one kernel (``b200_triplane_nerf``,
csrc/kernels/triplane.cu) that generates the lattice points itself; linears and attention go
through the usual ops. Tensor names follow the public ``stabilityai/TripoSR`` checkpoint.

Reference: src/HartsyInference.ThreeD/Models/TripoSr/ (TripoSrConfig.cs, TripoSrTransformer.cs,
TriplaneNerfDecoder.cs), Pipelines/TripoSrPipeline.cs, Geometry/Ops/GridSampler.cs.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch

from ... import ops
from ...ops import _native as N
from ..dit.common import WeightFactory
from ..encoders.vit import VitConfig, VitEncoder


@dataclass(frozen=True)
class TripoSrConfig:
    triplane_channels: int = 40
    plane_size: int = 32
    num_channels: int = 1024
    width: int = 1024
    depth: int = 16
    heads: int = 16
    head_dim: int = 64
    cross_dim: int = 768
    norm_groups: int = 32
    nerf_hidden: int = 64
    nerf_mid_layers: int = 8
    radius: float = 0.87
    density_bias: float = -1.0
    density_threshold: float = 25.0
    grid_resolution: int = 256
    image_size: int = 512
    vit: VitConfig = VitConfig(kind="vit", image_size=224, patch=16, width=768, layers=12, heads=12, ffn=3072, eps=1e-12,
                               activation="gelu")


TRIPOSR = TripoSrConfig()


def tiny_triposr() -> TripoSrConfig:
    return TripoSrConfig(triplane_channels=8, plane_size=4, num_channels=64, width=64, depth=2, heads=2, head_dim=32,
                         cross_dim=64, norm_groups=8, nerf_hidden=64, nerf_mid_layers=2, grid_resolution=24, image_size=64,
                         vit=VitConfig(kind="vit", image_size=64, patch=16, width=64, layers=2, heads=2, ffn=128, eps=1e-12,
                                       activation="gelu"))


def sample_triplane(planes: torch.Tensor, points: torch.Tensor, radius: float) -> torch.Tensor:
    """fp32 statement of the plane lookup: planes [3, C, H, W], points [N, 3] in [-R, R] -> [N, 3 C]
    (plane-major). ``grid_sample`` with bilinear weights, zero padding, align_corners = False."""
    p = points.float() / radius
    idx = torch.stack([p[:, [0, 1]], p[:, [0, 2]], p[:, [1, 2]]], 0)                  # [3, N, 2]
    f = torch.nn.functional.grid_sample(planes.float(), idx[:, None], mode="bilinear", padding_mode="zeros", align_corners=False)
    return f[:, :, 0].permute(2, 0, 1).reshape(points.shape[0], -1)                  # [N, 3 * C]


class TripoSr:
    def __init__(self, cfg: TripoSrConfig = TRIPOSR, device="cpu", get: Optional[Callable[[str], Optional[torch.Tensor]]] = None,
                 seed: int = 0):
        self.cfg, self.device = cfg, torch.device(device)
        f = WeightFactory(self.device, False, get=get, seed=seed)
        W, C = cfg.width, cfg.num_channels
        vget = None if get is None else (lambda n: get("image_tokenizer.model." + n))
        self.image_tokenizer = VitEncoder(cfg.vit, self.device, get=vget, seed=seed, prefix="")
        self.tokens = f.tensor("tokenizer.embeddings", 3, C, cfg.plane_size, cfg.plane_size).reshape(3, C, cfg.plane_size, cfg.plane_size)
        self.gn = (f.tensor("backbone.norm.weight", C, ones=True), f.tensor("backbone.norm.bias", C, zeros=True))
        self.proj_in = f.linear("backbone.proj_in", W, C)
        self.proj_out = f.linear("backbone.proj_out", C, W)
        self.blocks = []
        for i in range(cfg.depth):
            p = f"backbone.transformer_blocks.{i}."
            ln = lambda n: (f.tensor(p + n + ".weight", W, ones=True), f.tensor(p + n + ".bias", W, zeros=True))
            self.blocks.append(dict(
                n1=ln("norm1"), n2=ln("norm2"), n3=ln("norm3"),
                qkv=f.linear([p + "attn1.to_q", p + "attn1.to_k", p + "attn1.to_v"], [W, W, W], W, bias=False),
                o1=f.linear(p + "attn1.to_out.0", W, W),
                q2=f.linear(p + "attn2.to_q", W, W, bias=False),
                kv2=f.linear([p + "attn2.to_k", p + "attn2.to_v"], [W, W], cfg.cross_dim, bias=False),
                o2=f.linear(p + "attn2.to_out.0", W, W),
                ff_in=f.linear(p + "ff.net.0.proj", 8 * W, W), ff_out=f.linear(p + "ff.net.2", W, 4 * W)))
        tc = cfg.triplane_channels
        self.up_w = f.tensor("post_processor.upsample.weight", C, tc, 2, 2).reshape(C, tc, 2, 2)     # ConvTranspose2d [in, out, 2, 2]
        self.up_b = f.tensor("post_processor.upsample.bias", tc, zeros=True)
        h = cfg.nerf_hidden
        assert h == 64, "the fused field kernel is built for a hidden width of 64"
        mlp = [f.linear("decoder.layers.0", h, 3 * tc)]
        for i in range(cfg.nerf_mid_layers):
            mlp.append(f.linear(f"decoder.layers.{2 * (i + 1)}", h, h))
        mlp.append(f.linear(f"decoder.layers.{2 * (cfg.nerf_mid_layers + 1)}", 4, h))
        # the field decoder runs in fp32
        self.mlp_w = [m.weight.float().contiguous() for m in mlp]
        self.mlp_b = [m.bias.float().contiguous() for m in mlp]
        if cfg.nerf_mid_layers:
            self.mid_w = torch.stack(self.mlp_w[1:-1]).contiguous()
            self.mid_b = torch.stack(self.mlp_b[1:-1]).contiguous()
        else:
            self.mid_w = torch.zeros(0, h, h, device=self.device)
            self.mid_b = torch.zeros(0, h, device=self.device)

    # ------------------------------------------------------------------------------- image -> triplane
    def _ln(self, x, wb):
        return ops.norm(x, wb[0], bias=wb[1], layernorm=True, eps=1e-5)[0]

    @torch.no_grad()
    def triplane(self, image: torch.Tensor) -> torch.Tensor:
        """image [3, S, S] in [0, 1] (already composited on grey) -> planes [3, C_t, 2 P, 2 P] fp32."""
        cfg, dt = self.cfg, torch.bfloat16
        mean = torch.tensor([0.485, 0.456, 0.406], device=self.device)[:, None, None]
        std = torch.tensor([0.229, 0.224, 0.225], device=self.device)[:, None, None]
        ctx = self.image_tokenizer.hidden_states((image.to(self.device).float() - mean) / std)              # [1 + n, 768]
        P, C, W = cfg.plane_size, cfg.num_channels, cfg.width
        tok = self.tokens.float().permute(1, 0, 2, 3).reshape(C, 3 * P * P)                                   # [C, N]
        # GroupNorm over (channels of a group, all tokens)
        g = tok.reshape(cfg.norm_groups, -1)
        g = (g - g.mean(1, keepdim=True)) * torch.rsqrt(g.var(1, unbiased=False, keepdim=True) + 1e-6)
        x = (g.reshape(C, -1) * self.gn[0].float()[:, None] + self.gn[1].float()[:, None]).t().contiguous().to(dt)   # [N, C]
        x = ops.linear(x, self.proj_in)
        n, d, H = x.shape[0], cfg.head_dim, cfg.heads
        for b in self.blocks:
            q, k, v = ops.dit_qkv(ops.linear(self._ln(x, b["n1"]), b["qkv"]), H, H, d)
            x = ops.linear(ops.attention(q, k, v, causal=False).reshape(n, -1), b["o1"], residual=x)
            q2 = ops.linear(self._ln(x, b["n2"]), b["q2"]).reshape(n, H, d)
            kv = ops.linear(ctx, b["kv2"]).reshape(ctx.shape[0], 2, H, d)
            a = ops.attention(q2, kv[:, 0].contiguous(), kv[:, 1].contiguous(), causal=False).reshape(n, -1)
            x = ops.linear(a, b["o2"], residual=x)
            hgl = ops.linear(self._ln(x, b["n3"]), b["ff_in"]).float()                                       # GEGLU: value | gate
            val, gate = hgl[:, : 4 * W], hgl[:, 4 * W:]
            x = ops.linear((val * torch.nn.functional.gelu(gate)).to(dt), b["ff_out"], residual=x)
        x = ops.linear(x, self.proj_out).float().t() + tok                                                     # [C, N] + residual
        planes = x.reshape(C, 3, P, P).permute(1, 0, 2, 3)                                                      # [3, C, P, P]
        up = torch.nn.functional.conv_transpose2d(planes, self.up_w.float(), self.up_b.float(), stride=2)
        return up.contiguous()                                                                                  # [3, C_t, 2P, 2P]

    # ------------------------------------------------------------------------------- field decode
    @torch.no_grad()
    def field(self, planes: torch.Tensor, points: Optional[torch.Tensor] = None, resolution: int = 0) -> torch.Tensor:
        """[density_raw, r_raw, g_raw, b_raw] fp32 per point: for explicit ``points`` [N, 3], or for the
        ``resolution``^3 lattice over [-R, R]^3 (x outermost, z innermost, end points included)."""
        cfg = self.cfg
        if points is None:
            n = resolution ** 3
        else:
            points = points.to(self.device).float().contiguous()
            n = points.shape[0]
        if planes.is_cuda:
            out = torch.empty(n, 4, dtype=torch.float32, device=self.device)
            _, c, h, w = planes.shape
            N.check(N.lib().b200_triplane_nerf(planes.data_ptr(), c, h, w, N.ptr(points), 0, int(resolution), float(cfg.radius), n,
                                               self.mlp_w[0].data_ptr(), self.mlp_b[0].data_ptr(), self.mid_w.data_ptr(),
                                               self.mid_b.data_ptr(), cfg.nerf_mid_layers, self.mlp_w[-1].data_ptr(),
                                               self.mlp_b[-1].data_ptr(), out.data_ptr(), N.stream()), "b200_triplane_nerf")
            return out
        if points is None:
            ax = torch.linspace(-cfg.radius, cfg.radius, resolution)
            points = torch.stack(torch.meshgrid(ax, ax, ax, indexing="ij"), -1).reshape(-1, 3)
        outs = []
        for c0 in range(0, n, 1 << 18):
            hcur = sample_triplane(planes, points[c0:c0 + (1 << 18)], cfg.radius)
            for i, (w_, b_) in enumerate(zip(self.mlp_w, self.mlp_b)):
                hcur = hcur @ w_.t() + b_
                if i + 1 < len(self.mlp_w):
                    hcur = torch.nn.functional.silu(hcur)
            outs.append(hcur)
        return torch.cat(outs)

    def density(self, raw: torch.Tensor) -> torch.Tensor:
        return torch.exp(raw[:, 0] + self.cfg.density_bias)

    @torch.no_grad()
    def extract_mesh(self, planes: torch.Tensor, resolution: Optional[int] = None, threshold: Optional[float] = None):
        """-> (vertices [V, 3] in [-R, R], faces [F, 3], colours [V, 3] in [0, 1])."""
        from ...threed.marching_cubes import marching_cubes
        cfg = self.cfg
        res = resolution or cfg.grid_resolution
        dens = self.density(self.field(planes, resolution=res)).reshape(res, res, res)
        step = 2 * cfg.radius / (res - 1)
        # inside = density above the threshold: extract the iso-surface of (threshold - density)
        verts, faces = marching_cubes((threshold if threshold is not None else cfg.density_threshold) - dens, 0.0,
                                      spacing=(step, step, step), origin=(-cfg.radius,) * 3)
        if verts.shape[0] == 0:
            return verts, faces, torch.zeros(0, 3)
        rgb = torch.sigmoid(self.field(planes, points=verts.to(self.device))[:, 1:4])
        return verts, faces, rgb
