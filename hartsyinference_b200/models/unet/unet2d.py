"""Conditional 2-D U-Net of Stable Diffusion 1.5 and SDXL (diffusers ``UNet2DConditionModel`` layout).

Structure (all levels share it; the configs differ in depth and widths):

* time embedding: sinusoidal code of the timestep (cosines first) -> Linear, SiLU, Linear. SDXL adds a
  second embedding of its micro-conditioning (the pooled text vector next to six sinusoid-coded
  size / crop numbers) to it;
* down path: ``conv_in``, then per level ``layers_per_block`` pairs of (ResNet block, transformer block
  if the level attends) and a stride-2 convolution between levels; every output is kept as a skip;
* middle: ResNet, transformer, ResNet at the deepest width;
* up path: per level ``layers_per_block + 1`` ResNet blocks, each over the concatenation of the running
  tensor and the most recent skip, with the level's transformer after each, then nearest 2x + 3x3
  convolution between levels; GroupNorm, SiLU, ``conv_out``.

A ResNet block is GroupNorm-SiLU-conv twice with the projected time embedding added in between and a
1x1 shortcut when the width changes. A transformer block is GroupNorm, projection in (1x1 conv in
SD 1.5, Linear in SDXL), ``depth`` layers of (LayerNorm, self-attention, LayerNorm, cross-attention
into the text states, LayerNorm, GEGLU feed-forward), projection out, residual.

The linear layers of the transformer blocks (almost all FLOPs of SDXL at 1024 px) run on the
tcgen05 GEMM on a CUDA device (``ops.linear``), attention through the framework's attention op when the
head dim allows and torch's fused attention otherwise; convolutions and GroupNorm go through cuDNN.

Reference: src/HartsyInference.Diffusion/Models/Denoisers/UNet.cs, UNetConfig.cs, UNetBlocks/
(DownBlock, UpBlock, UNetResNetBlock, CrossAttentionBlock, TimestepEmbedding, AdditionEmbedding).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.nn.functional as F

from ... import ops
from ...ops import LinearWeight


@dataclass(frozen=True)
class UNetConfig:
    in_channels: int = 4
    out_channels: int = 4
    block_out_channels: tuple = (320, 640, 1280, 1280)
    layers_per_block: int = 2
    cross_attention_dim: int = 768
    num_heads: tuple = (8, 8, 8, 8)                       # heads per level (diffusers calls this attention_head_dim)
    down_attention: tuple = (True, True, True, False)
    up_attention: tuple = (False, True, True, True)
    transformer_layers: tuple = (1, 1, 1, 1)
    norm_groups: int = 32
    norm_eps: float = 1e-5
    linear_projection: bool = False
    addition_embed_dim: int = 0                           # width of the micro-conditioning vector (0: none)
    addition_time_embed_dim: int = 256

    @property
    def time_embed_dim(self) -> int:
        return 4 * self.block_out_channels[0]


SD15 = UNetConfig()
SDXL_BASE = UNetConfig(block_out_channels=(320, 640, 1280), cross_attention_dim=2048, num_heads=(5, 10, 20),
                       down_attention=(False, True, True), up_attention=(True, True, False), transformer_layers=(1, 2, 10),
                       linear_projection=True, addition_embed_dim=2816)
SDXL_REFINER = UNetConfig(block_out_channels=(384, 768, 1536, 1536), cross_attention_dim=1280, num_heads=(6, 12, 24, 24),
                          down_attention=(False, True, True, False), up_attention=(False, True, True, False),
                          transformer_layers=(4, 4, 4, 4), linear_projection=True, addition_embed_dim=2560)


def tiny_unet(sdxl: bool = False) -> UNetConfig:
    if sdxl:
        return UNetConfig(block_out_channels=(32, 64), cross_attention_dim=48, num_heads=(2, 4), down_attention=(False, True),
                          up_attention=(True, False), transformer_layers=(1, 2), norm_groups=8, linear_projection=True,
                          addition_embed_dim=6 * 8 + 24, addition_time_embed_dim=8, layers_per_block=1)
    return UNetConfig(block_out_channels=(32, 64), cross_attention_dim=48, num_heads=(2, 2), down_attention=(True, False),
                      up_attention=(False, True), transformer_layers=(1, 1), norm_groups=8, layers_per_block=1)


def unet_from_hf(d: dict) -> UNetConfig:
    ch = tuple(d.get("block_out_channels", (320, 640, 1280, 1280)))
    n = len(ch)
    heads = d.get("num_attention_heads") or d.get("attention_head_dim", 8)
    heads = tuple(heads) if isinstance(heads, (list, tuple)) else (heads,) * n
    tl = d.get("transformer_layers_per_block", 1)
    tl = tuple(tl) if isinstance(tl, (list, tuple)) else (tl,) * n
    down = tuple("CrossAttn" in t for t in d.get("down_block_types", ("CrossAttnDownBlock2D",) * (n - 1) + ("DownBlock2D",)))
    up = tuple("CrossAttn" in t for t in d.get("up_block_types", ("UpBlock2D",) + ("CrossAttnUpBlock2D",) * (n - 1)))
    add = int(d.get("projection_class_embeddings_input_dim") or 0) if d.get("addition_embed_type") == "text_time" else 0
    return UNetConfig(in_channels=d.get("in_channels", 4), out_channels=d.get("out_channels", 4), block_out_channels=ch,
                      layers_per_block=d.get("layers_per_block", 2), cross_attention_dim=d.get("cross_attention_dim", 768),
                      num_heads=heads, down_attention=down, up_attention=up, transformer_layers=tl,
                      norm_groups=d.get("norm_num_groups", 32), norm_eps=float(d.get("norm_eps", 1e-5)),
                      linear_projection=bool(d.get("use_linear_projection", False)), addition_embed_dim=add,
                      addition_time_embed_dim=int(d.get("addition_time_embed_dim") or 256))


def sinusoid(values: torch.Tensor, dim: int) -> torch.Tensor:
    """[N] -> [N, dim]: cosines of value * 10000^(-i / half) first, then the sines."""
    half = dim // 2
    f = torch.exp(-math.log(10000.0) * torch.arange(half, dtype=torch.float32, device=values.device) / half)
    a = values.float()[:, None] * f[None]
    return torch.cat([a.cos(), a.sin()], -1)


class UNet2D:
    """``get(name)`` returns checkpoint tensors by their diffusers names (random weights without it)."""

    def __init__(self, cfg: UNetConfig = SD15, device="cpu", get: Optional[Callable[[str], Optional[torch.Tensor]]] = None,
                 seed: int = 0, dtype: Optional[torch.dtype] = None):
        self.cfg, self.device = cfg, torch.device(device)
        self.dtype = dtype or (torch.bfloat16 if self.device.type == "cuda" else torch.float32)
        self._get, self._g = get, torch.Generator().manual_seed(seed)
        self._w: dict = {}
        self._lin: dict = {}
        self._ip: Optional[dict] = None

    def cross_attention_paths(self) -> list[str]:
        """Every cross-attention layer in the order adapters index them: down blocks, up blocks, middle block."""
        cfg = self.cfg
        out = []
        for i in range(len(cfg.block_out_channels)):
            if cfg.down_attention[i]:
                out += [f"down_blocks.{i}.attentions.{j}.transformer_blocks.{k}.attn2" for j in range(cfg.layers_per_block)
                        for k in range(cfg.transformer_layers[i])]
        depth = list(reversed(cfg.transformer_layers))
        for i in range(len(cfg.block_out_channels)):
            if cfg.up_attention[i]:
                out += [f"up_blocks.{i}.attentions.{j}.transformer_blocks.{k}.attn2" for j in range(cfg.layers_per_block + 1)
                        for k in range(depth[i])]
        out += [f"mid_block.attentions.0.transformer_blocks.{k}.attn2" for k in range(cfg.transformer_layers[-1])]
        return out

    # ------------------------------------------------------------------------------ weights
    def _tensor(self, name: str, shape: tuple, kind: str = "weight"):
        t = self._w.get(name)
        if t is None:
            raw = self._get(name) if self._get is not None else None
            if raw is None:
                if self._get is not None:
                    raise KeyError(name)
                if kind == "ones":
                    raw = torch.ones(shape)
                elif kind == "zeros":
                    raw = torch.zeros(shape)
                else:
                    fan = 1
                    for s in shape[1:]:
                        fan *= s
                    raw = torch.randn(shape, generator=self._g) * (1.0 / max(fan, 1)) ** 0.5
            t = raw.reshape(shape).to(self.device).to(self.dtype)
            self._w[name] = t
        return t

    def _linear(self, x: torch.Tensor, name: str, n: int, k: int, bias: bool = True) -> torch.Tensor:
        lw = self._lin.get(name)
        if lw is None:
            lw = LinearWeight(self._tensor(name + ".weight", (n, k)).contiguous(), None,
                              self._tensor(name + ".bias", (n,), "zeros") if bias else None)
            self._lin[name] = lw
        if x.is_cuda and x.dtype == torch.bfloat16 and k % 64 == 0 and n % 16 == 0:
            shape = x.shape
            return ops.linear(x.reshape(-1, k).contiguous(), lw).reshape(*shape[:-1], n)
        return F.linear(x, lw.weight, lw.bias)

    def _conv(self, x, name: str, co: int, ci: int, k: int, stride: int = 1):
        return F.conv2d(x, self._tensor(name + ".weight", (co, ci, k, k)), self._tensor(name + ".bias", (co,), "zeros"),
                        stride=stride, padding=k // 2)

    def _gn(self, x, name: str, c: int, eps: Optional[float] = None):
        return F.group_norm(x, self.cfg.norm_groups, self._tensor(name + ".weight", (c,), "ones"),
                            self._tensor(name + ".bias", (c,), "zeros"), self.cfg.norm_eps if eps is None else eps)

    def _ln(self, x, name: str, c: int):
        return F.layer_norm(x, (c,), self._tensor(name + ".weight", (c,), "ones"), self._tensor(name + ".bias", (c,), "zeros"), 1e-5)

    # ------------------------------------------------------------------------------ blocks
    def _resnet(self, x, emb_act, p: str, ci: int, co: int):
        h = self._conv(F.silu(self._gn(x, p + ".norm1", ci)), p + ".conv1", co, ci, 3)
        h = h + self._linear(emb_act, p + ".time_emb_proj", co, self.cfg.time_embed_dim)[:, :, None, None]
        h = self._conv(F.silu(self._gn(h, p + ".norm2", co)), p + ".conv2", co, co, 3)
        if ci != co:
            x = self._conv(x, p + ".conv_shortcut", co, ci, 1)
        return x + h

    def _attention(self, x, ctx, p: str, c: int, heads: int, kdim: int):
        b, t, _ = x.shape
        d = c // heads
        q = self._linear(x, p + ".to_q", c, c, bias=False).view(b, t, heads, d).transpose(1, 2)
        k = self._linear(ctx, p + ".to_k", c, kdim, bias=False).view(b, ctx.shape[1], heads, d).transpose(1, 2)
        v = self._linear(ctx, p + ".to_v", c, kdim, bias=False).view(b, ctx.shape[1], heads, d).transpose(1, 2)
        o = F.scaled_dot_product_attention(q, k, v)
        ip = self._ip
        if ip is not None and p in ip["layers"]:
            # decoupled cross-attention: the same queries over keys / values projected from the image tokens
            wk, wv = ip["layers"][p]
            tok = ip["tokens"]
            ik = F.linear(tok, wk).view(b, tok.shape[1], heads, d).transpose(1, 2)
            iv = F.linear(tok, wv).view(b, tok.shape[1], heads, d).transpose(1, 2)
            o = o + ip["scale"] * F.scaled_dot_product_attention(q, ik, iv)
        return self._linear(o.transpose(1, 2).reshape(b, t, c), p + ".to_out.0", c, c)

    def _transformer(self, x, context, p: str, c: int, heads: int, depth: int):
        cfg = self.cfg
        b, _, h, w = x.shape
        res = x
        y = self._gn(x, p + ".norm", c, eps=1e-6)
        if cfg.linear_projection:
            y = self._linear(y.permute(0, 2, 3, 1).reshape(b, h * w, c), p + ".proj_in", c, c)
        else:
            y = self._conv(y, p + ".proj_in", c, c, 1).permute(0, 2, 3, 1).reshape(b, h * w, c)
        for i in range(depth):
            q = f"{p}.transformer_blocks.{i}"
            n1 = self._ln(y, q + ".norm1", c)
            y = y + self._attention(n1, n1, q + ".attn1", c, heads, c)
            y = y + self._attention(self._ln(y, q + ".norm2", c), context, q + ".attn2", c, heads, cfg.cross_attention_dim)
            f = self._linear(self._ln(y, q + ".norm3", c), q + ".ff.net.0.proj", 8 * c, c)
            val, gate = f.chunk(2, -1)
            y = y + self._linear(val * F.gelu(gate), q + ".ff.net.2", c, 4 * c)
        if cfg.linear_projection:
            y = self._linear(y, p + ".proj_out", c, c).reshape(b, h, w, c).permute(0, 3, 1, 2)
        else:
            y = self._conv(y.reshape(b, h, w, c).permute(0, 3, 1, 2), p + ".proj_out", c, c, 1)
        return y + res

    # ------------------------------------------------------------------------------ forward
    def _embedding(self, b: int, timestep, pooled, time_ids) -> torch.Tensor:
        cfg = self.cfg
        ch = cfg.block_out_channels
        t = torch.as_tensor(timestep, dtype=torch.float32, device=self.device).reshape(-1).expand(b)
        te = cfg.time_embed_dim
        emb = self._linear(sinusoid(t, ch[0]).to(self.dtype), "time_embedding.linear_1", te, ch[0])
        emb = self._linear(F.silu(emb), "time_embedding.linear_2", te, te)
        if cfg.addition_embed_dim:
            if pooled is None or time_ids is None:
                raise ValueError("this U-Net needs the pooled text vector and the size / crop numbers")
            ids = sinusoid(time_ids.to(self.device).reshape(-1), cfg.addition_time_embed_dim).reshape(b, -1)
            add = torch.cat([pooled.to(self.device).float(), ids], -1).to(self.dtype)
            assert add.shape[-1] == cfg.addition_embed_dim, (add.shape, cfg.addition_embed_dim)
            a = self._linear(add, "add_embedding.linear_1", te, cfg.addition_embed_dim)
            emb = emb + self._linear(F.silu(a), "add_embedding.linear_2", te, te)
        return F.silu(emb)

    def _down_and_mid(self, x, emb_act, context, after_conv_in: Optional[torch.Tensor] = None):
        """conv_in, the down blocks and the middle block: (skips as (tensor, channels), middle output)."""
        cfg = self.cfg
        ch = cfg.block_out_channels
        x = self._conv(x, "conv_in", ch[0], cfg.in_channels, 3)
        if after_conv_in is not None:
            x = x + after_conv_in
        skips = [(x, ch[0])]
        prev = ch[0]
        for i, c in enumerate(ch):
            for j in range(cfg.layers_per_block):
                x = self._resnet(x, emb_act, f"down_blocks.{i}.resnets.{j}", prev, c)
                prev = c
                if cfg.down_attention[i]:
                    x = self._transformer(x, context, f"down_blocks.{i}.attentions.{j}", c, cfg.num_heads[i], cfg.transformer_layers[i])
                skips.append((x, c))
            if i < len(ch) - 1:
                x = self._conv(x, f"down_blocks.{i}.downsamplers.0.conv", c, c, 3, stride=2)
                skips.append((x, c))
        top = ch[-1]
        x = self._resnet(x, emb_act, "mid_block.resnets.0", top, top)
        x = self._transformer(x, context, "mid_block.attentions.0", top, cfg.num_heads[-1], cfg.transformer_layers[-1])
        x = self._resnet(x, emb_act, "mid_block.resnets.1", top, top)
        return skips, x

    @torch.no_grad()
    def forward(self, latents: torch.Tensor, timestep: torch.Tensor, context: torch.Tensor,
                pooled: Optional[torch.Tensor] = None, time_ids: Optional[torch.Tensor] = None,
                down_residuals: Optional[list] = None, mid_residual: Optional[torch.Tensor] = None,
                image_tokens: Optional[torch.Tensor] = None, image_scale: float = 1.0) -> torch.Tensor:
        """latents [B, C, h, w], timestep [B] (or scalar), context [B, L, cross_attention_dim]; SDXL also takes
        ``pooled`` [B, P] and ``time_ids`` [B, 6] (original size, crop offset, target size). ``down_residuals`` /
        ``mid_residual`` (a ControlNet's outputs) are added to the skip connections and the middle block's
        output; ``image_tokens`` [B, n, cross_attention_dim] go through the image adapter installed with
        :func:`install_ip_adapter`. Returns the prediction [B, C, h, w] in fp32."""
        cfg = self.cfg
        ch = cfg.block_out_channels
        x = latents.to(self.device).to(self.dtype)
        b = x.shape[0]
        context = context.to(self.device).to(self.dtype)
        emb_act = self._embedding(b, timestep, pooled, time_ids)
        if self._ip is not None:
            self._ip["tokens"] = None if image_tokens is None else image_tokens.to(self.device).to(self.dtype)
            self._ip["scale"] = float(image_scale)
        ip_saved = self._ip
        if image_tokens is None:
            self._ip = None
        try:
            skips, x = self._down_and_mid(x, emb_act, context)
            if down_residuals is not None:
                if len(down_residuals) != len(skips):
                    raise ValueError(f"{len(down_residuals)} residuals for {len(skips)} skip connections")
                skips = [(s + r.to(s.dtype), c) for (s, c), r in zip(skips, down_residuals)]
            if mid_residual is not None:
                x = x + mid_residual.to(x.dtype)
            top = ch[-1]
            rev = list(reversed(ch))
            heads, depth = list(reversed(cfg.num_heads)), list(reversed(cfg.transformer_layers))
            prev = top
            for i, c in enumerate(rev):
                for j in range(cfg.layers_per_block + 1):
                    skip, sc = skips.pop()
                    x = self._resnet(torch.cat([x, skip], 1), emb_act, f"up_blocks.{i}.resnets.{j}", prev + sc, c)
                    prev = c
                    if cfg.up_attention[i]:
                        x = self._transformer(x, context, f"up_blocks.{i}.attentions.{j}", c, heads[i], depth[i])
                if i < len(rev) - 1:
                    x = self._conv(F.interpolate(x, scale_factor=2.0, mode="nearest"), f"up_blocks.{i}.upsamplers.0.conv", c, c, 3)
        finally:
            self._ip = ip_saved
        x = F.silu(self._gn(x, "conv_norm_out", ch[0]))
        return self._conv(x, "conv_out", cfg.out_channels, ch[0], 3).float()


class ControlNet(UNet2D):
    """The U-Net's encoder half run on the same latents plus a conditioning picture: the picture [B, 3, 8h, 8w]
    goes through a small strided convolution stack (16, 32, 96, 256 channels, three stride-2 steps) and is added
    after ``conv_in``; every skip connection and the middle output pass through a zero-initialised 1 x 1
    convolution and are returned, scaled, for :meth:`UNet2D.forward` to add. Weights by the diffusers names
    (``controlnet_cond_embedding.*``, ``controlnet_down_blocks.N``, ``controlnet_mid_block``). Reference:
    src/HartsyInference.Diffusion/Adapters/ (ControlNet for U-Net models)."""

    HINT_CHANNELS = (16, 32, 96, 256)

    def _hint(self, cond: torch.Tensor) -> torch.Tensor:
        hc = self.HINT_CHANNELS
        p = "controlnet_cond_embedding"
        x = F.silu(self._conv(cond, p + ".conv_in", hc[0], cond.shape[1], 3))
        k = 0
        for i in range(len(hc) - 1):
            x = F.silu(self._conv(x, f"{p}.blocks.{k}", hc[i], hc[i], 3))
            x = F.silu(self._conv(x, f"{p}.blocks.{k + 1}", hc[i + 1], hc[i], 3, stride=2))
            k += 2
        return self._conv(x, p + ".conv_out", self.cfg.block_out_channels[0], hc[-1], 3)

    @torch.no_grad()
    def forward(self, latents, timestep, context, cond: torch.Tensor, pooled=None, time_ids=None, scale: float = 1.0):
        """-> (down residuals, one per skip connection; middle residual), each already multiplied by ``scale``."""
        x = latents.to(self.device).to(self.dtype)
        emb_act = self._embedding(x.shape[0], timestep, pooled, time_ids)
        hint = self._hint(cond.to(self.device).to(self.dtype))
        skips, mid = self._down_and_mid(x, emb_act, context.to(self.device).to(self.dtype), after_conv_in=hint)
        down = [self._conv(s, f"controlnet_down_blocks.{i}", c, c, 1) * scale for i, (s, c) in enumerate(skips)]
        top = self.cfg.block_out_channels[-1]
        return down, self._conv(mid, "controlnet_mid_block", top, top, 1) * scale


def install_ip_adapter(unet: UNet2D, get: Callable[[str], Optional[torch.Tensor]]) -> Callable[[torch.Tensor], torch.Tensor]:
    """Attaches an image-prompt adapter (``ip_adapter.N.to_k_ip / to_v_ip`` per cross-attention layer, N = 2 i + 1 in
    the adapters' layer order; ``image_proj.proj`` + ``image_proj.norm``) to ``unet``. Returns the projector:
    CLIP image embedding [B, E] -> image tokens [B, n, cross_attention_dim] for ``forward(image_tokens=...)``.
    Reference: src/HartsyInference.Diffusion/Adapters/ (IP-Adapter)."""
    layers = {}
    for i, path in enumerate(unet.cross_attention_paths()):
        wk, wv = get(f"ip_adapter.{2 * i + 1}.to_k_ip.weight"), get(f"ip_adapter.{2 * i + 1}.to_v_ip.weight")
        if wk is None or wv is None:
            raise KeyError(f"ip_adapter.{2 * i + 1}.to_k_ip.weight")
        layers[path] = (wk.to(unet.device).to(unet.dtype), wv.to(unet.device).to(unet.dtype))
    unet._ip = {"layers": layers, "tokens": None, "scale": 1.0}
    pw, pb = get("image_proj.proj.weight").to(unet.device).float(), get("image_proj.proj.bias").to(unet.device).float()
    nw, nb = get("image_proj.norm.weight").to(unet.device).float(), get("image_proj.norm.bias").to(unet.device).float()
    dim = unet.cfg.cross_attention_dim

    def project(image_embeds: torch.Tensor) -> torch.Tensor:
        e = image_embeds.to(unet.device).float()
        tok = F.linear(e, pw, pb).view(e.shape[0], -1, dim)
        return F.layer_norm(tok, (dim,), nw, nb).to(unet.dtype)

    return project
