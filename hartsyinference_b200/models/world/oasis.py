"""Oasis-500M action-conditioned world model: autoregressive in time, diffusion in space.

Three parts, all transformers:

* ``OasisVae``: a ViT autoencoder. 20 x 20 RGB patches -> 6 encoder blocks -> LayerNorm -> linear
  Gaussian bottleneck (the mean is used) of 16 channels per patch; 16 -> width -> 12 decoder blocks ->
  LayerNorm -> linear patch predictor. Blocks: affine LayerNorm, fused-QKV self-attention with a 2-d
  axial rotary embedding ("pixel" frequencies) over the first half of every head, 4x GELU MLP.
* ``OasisDit``: the denoiser over a window of latent frames [T, 16, h, w]. 2 x 2 latent patches, 16
  blocks of a spatial half (attention among the tokens of one frame, 2-d axial rotary embedding) and a
  temporal half (CAUSAL attention along time at every location, 1-d rotary embedding), each half with
  its own adaLN-zero modulation from the frame's conditioning ``time_embed(noise level of the frame) +
  linear(action of the frame)``: every frame carries its own noise level (diffusion forcing).
* ``OasisWorld``: the sampler. A new frame starts as clamped Gaussian noise and is denoised with 10
  v-prediction DDIM steps over a sigmoid beta schedule while the frames already committed are held at
  a small fixed noise level and stay as they are; the window slides at 32 frames.

On a CUDA device the linear layers run on the tcgen05 GEMM (``ops.linear``) in bf16 and the rest in
tensor ops; head dim 64 attention goes through torch's fused attention.

Reference: src/HartsyInference.World/Pipelines/OasisPipeline.cs,
src/HartsyInference.Diffusion/Models/Denoisers/OasisDit.cs (+ DiTBlocks/OasisSpatioTemporalBlock.cs),
src/HartsyInference.Diffusion/Models/Vae/OasisVitVae.cs; tensor names of the released checkpoint
(``x_embedder``, ``t_embedder``, ``external_cond``, ``blocks.N.{s,t}_*``, ``final_layer``; VAE:
``patch_embed``, ``encoder.N``, ``enc_norm``, ``quant_conv``, ``post_quant_conv``, ``decoder.N``,
``dec_norm``, ``predictor``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.nn.functional as F

from ... import ops
from ...ops import LinearWeight

ACTION_DIM = 25               # 23 keys / buttons + 2 camera deltas
SCALING = 0.07843137255       # latents are multiplied by 20 / 255 before the denoiser sees them


@dataclass(frozen=True)
class OasisConfig:
    # denoiser
    latent_channels: int = 16
    patch: int = 2
    hidden: int = 1024
    depth: int = 16
    heads: int = 16
    mlp_ratio: float = 4.0
    action_dim: int = ACTION_DIM
    max_frames: int = 32
    freq_dim: int = 256
    spatial_max_freq: float = 256.0
    # autoencoder
    vae_patch: int = 20
    vae_width: int = 1024
    vae_heads: int = 16
    vae_enc_depth: int = 6
    vae_dec_depth: int = 12
    # sampler
    train_steps: int = 1000
    ddim_steps: int = 10
    stabilization_level: int = 15
    noise_abs_max: float = 20.0


def tiny_oasis(**kw) -> OasisConfig:
    base = dict(hidden=64, depth=2, heads=2, vae_patch=4, vae_width=64, vae_heads=2, vae_enc_depth=1, vae_dec_depth=2,
                max_frames=4, ddim_steps=3, freq_dim=32)
    base.update(kw)
    return OasisConfig(**base)


# ---------------------------------------------------------------------------------- rotary tables
def _interleave2(t: torch.Tensor) -> torch.Tensor:
    return t.repeat_interleave(2, dim=-1)


def axial_freqs_2d(h: int, w: int, dim_per_axis: int, max_freq: float) -> torch.Tensor:
    """[h * w, 2 * dim_per_axis] rotation angles: positions on [-1, 1] along each axis times
    ``linspace(1, max_freq / 2, dim_per_axis / 2) * pi``, every angle used for a pair of adjacent dims;
    row angles first, then column angles."""
    f = torch.linspace(1.0, max_freq / 2, dim_per_axis // 2) * math.pi
    ay = _interleave2(torch.linspace(-1, 1, h)[:, None] * f[None])          # [h, dim_per_axis]
    ax = _interleave2(torch.linspace(-1, 1, w)[:, None] * f[None])
    return torch.cat([ay[:, None, :].expand(h, w, -1), ax[None, :, :].expand(h, w, -1)], -1).reshape(h * w, -1)


def temporal_freqs(t: int, dim: int, theta: float = 10000.0) -> torch.Tensor:
    f = 1.0 / (theta ** (torch.arange(0, dim, 2).float() / dim))
    return _interleave2(torch.arange(t).float()[:, None] * f[None])            # [t, dim]


def apply_rotary(x: torch.Tensor, angles: torch.Tensor) -> torch.Tensor:
    """Rotates adjacent pairs of the first ``angles.shape[-1]`` dims of ``x`` [..., seq, d]; angles [seq, r]."""
    r = angles.shape[-1]
    xr, rest = x[..., :r].float(), x[..., r:]
    x1, x2 = xr[..., 0::2], xr[..., 1::2]
    half = torch.stack([-x2, x1], -1).flatten(-2)
    out = xr * angles.cos() + half * angles.sin()
    return torch.cat([out.to(x.dtype), rest], -1)


class _Weights:
    """Checkpoint access: ``get(name)`` by released names, or seeded random tensors for synthetic models."""

    def __init__(self, device, dtype, get, seed: int, prefix: str = ""):
        self.device, self.dtype, self.get, self.prefix = torch.device(device), dtype, get, prefix
        self.g = torch.Generator().manual_seed(seed)
        self.lin: dict = {}
        self.vec: dict = {}

    def linear(self, name: str, n: int, k: int, bias: bool = True, zero: bool = False) -> LinearWeight:
        lw = self.lin.get(name)
        if lw is None:
            w = self.get(self.prefix + name + ".weight") if self.get else None
            b = self.get(self.prefix + name + ".bias") if (self.get and bias) else None
            if w is None:
                if self.get is not None:
                    raise KeyError(self.prefix + name + ".weight")
                w = torch.zeros(n, k) if zero else torch.randn(n, k, generator=self.g) * (1.0 / k) ** 0.5
                b = (torch.randn(n, generator=self.g) * 0.02) if bias else None
            w = w.reshape(n, k)
            lw = LinearWeight(w.to(self.dtype).to(self.device).contiguous(), None,
                              None if b is None else b.to(self.dtype).to(self.device))
            self.lin[name] = lw
        return lw

    def vector(self, name: str, n: int, ones: bool = False) -> torch.Tensor:
        v = self.vec.get(name)
        if v is None:
            t = self.get(self.prefix + name) if self.get else None
            if t is None:
                if self.get is not None:
                    raise KeyError(self.prefix + name)
                t = torch.ones(n) if ones else torch.zeros(n)
            v = t.float().to(self.device)
            self.vec[name] = v
        return v


def _linear(x: torch.Tensor, lw: LinearWeight) -> torch.Tensor:
    shape = x.shape
    if x.is_cuda and x.dtype == torch.bfloat16 and shape[-1] % 64 == 0 and lw.out_features % 16 == 0:
        return ops.linear(x.reshape(-1, shape[-1]).contiguous(), lw).reshape(*shape[:-1], lw.out_features)
    return F.linear(x, lw.weight, lw.bias)


def _mha(q, k, v, causal: bool = False):
    return F.scaled_dot_product_attention(q, k, v, is_causal=causal)


# ---------------------------------------------------------------------------------- autoencoder
class OasisVae:
    def __init__(self, cfg: OasisConfig, device="cpu", get: Optional[Callable] = None, seed: int = 0,
                 dtype: Optional[torch.dtype] = None):
        self.cfg, self.device = cfg, torch.device(device)
        self.dtype = dtype or (torch.bfloat16 if self.device.type == "cuda" else torch.float32)
        self.w = _Weights(device, self.dtype, get, seed + 100)

    def _block(self, x: torch.Tensor, p: str, angles: torch.Tensor) -> torch.Tensor:
        c, w = self.cfg, self.w
        d, heads = c.vae_width, c.vae_heads
        b, s, _ = x.shape
        y = F.layer_norm(x.float(), (d,), w.vector(p + ".norm1.weight", d, True), w.vector(p + ".norm1.bias", d)).to(x.dtype)
        qkv = _linear(y, w.linear(p + ".attn.qkv", 3 * d, d)).view(b, s, 3, heads, d // heads).permute(2, 0, 3, 1, 4)
        q, k = apply_rotary(qkv[0], angles), apply_rotary(qkv[1], angles)
        o = _mha(q, k, qkv[2]).transpose(1, 2).reshape(b, s, d)
        x = x + _linear(o, w.linear(p + ".attn.proj", d, d))
        y = F.layer_norm(x.float(), (d,), w.vector(p + ".norm2.weight", d, True), w.vector(p + ".norm2.bias", d)).to(x.dtype)
        hid = int(d * 4)
        return x + _linear(F.gelu(_linear(y, w.linear(p + ".mlp.fc1", hid, d))), w.linear(p + ".mlp.fc2", d, hid))

    def _angles(self, gh: int, gw: int) -> torch.Tensor:
        # the first half of every head is rotated: a quarter of the head per axis
        per_axis = self.cfg.vae_width // self.cfg.vae_heads // 4
        return axial_freqs_2d(gh, gw, per_axis, self.cfg.spatial_max_freq).to(self.device)

    @torch.no_grad()
    def encode(self, rgb: torch.Tensor) -> torch.Tensor:
        """rgb [B, 3, H, W] in [-1, 1] -> posterior mean [B, 16, H / p, W / p] (unscaled)."""
        c, w, p = self.cfg, self.w, self.cfg.vae_patch
        b, _, hh, ww = rgb.shape
        gh, gw = hh // p, ww // p
        x = rgb.to(self.device).to(self.dtype).reshape(b, 3, gh, p, gw, p).permute(0, 2, 4, 1, 3, 5).reshape(b, gh * gw, 3 * p * p)
        x = _linear(x, w.linear("patch_embed.proj", c.vae_width, 3 * p * p))
        ang = self._angles(gh, gw)
        for i in range(c.vae_enc_depth):
            x = self._block(x, f"encoder.{i}", ang)
        d = c.vae_width
        x = F.layer_norm(x.float(), (d,), w.vector("enc_norm.weight", d, True), w.vector("enc_norm.bias", d)).to(x.dtype)
        moments = _linear(x, w.linear("quant_conv", 2 * c.latent_channels, d))
        mean = moments[..., :c.latent_channels].float()
        return mean.reshape(b, gh, gw, c.latent_channels).permute(0, 3, 1, 2).contiguous()

    @torch.no_grad()
    def decode(self, z: torch.Tensor) -> torch.Tensor:
        """z [B, 16, h, w] (unscaled) -> rgb [B, 3, h p, w p] in [-1, 1] (fp32)."""
        c, w, p = self.cfg, self.w, self.cfg.vae_patch
        b, ch, gh, gw = z.shape
        d = c.vae_width
        x = z.to(self.device).to(self.dtype).permute(0, 2, 3, 1).reshape(b, gh * gw, ch)
        x = _linear(x, w.linear("post_quant_conv", d, ch))
        ang = self._angles(gh, gw)
        for i in range(c.vae_dec_depth):
            x = self._block(x, f"decoder.{i}", ang)
        x = F.layer_norm(x.float(), (d,), w.vector("dec_norm.weight", d, True), w.vector("dec_norm.bias", d)).to(x.dtype)
        x = _linear(x, w.linear("predictor", 3 * p * p, d)).float()
        # patch vectors are channel-major: (channel, row in patch, column in patch)
        return x.reshape(b, gh, gw, 3, p, p).permute(0, 3, 1, 4, 2, 5).reshape(b, 3, gh * p, gw * p)


# ---------------------------------------------------------------------------------- denoiser
class OasisDit:
    def __init__(self, cfg: OasisConfig, device="cpu", get: Optional[Callable] = None, seed: int = 0,
                 dtype: Optional[torch.dtype] = None):
        self.cfg, self.device = cfg, torch.device(device)
        self.dtype = dtype or (torch.bfloat16 if self.device.type == "cuda" else torch.float32)
        self.w = _Weights(device, self.dtype, get, seed)
        self._tables: dict = {}

    def _time_embed(self, levels: torch.Tensor) -> torch.Tensor:
        c, w = self.cfg, self.w
        half = c.freq_dim // 2
        f = torch.exp(-math.log(10000.0) * torch.arange(half, dtype=torch.float32, device=self.device) / half)
        a = levels.float().to(self.device)[:, None] * f[None]
        e = torch.cat([a.cos(), a.sin()], -1).to(self.dtype)
        return _linear(F.silu(_linear(e, w.linear("t_embedder.mlp.0", c.hidden, c.freq_dim))), w.linear("t_embedder.mlp.2", c.hidden, c.hidden))

    def _rope(self, t: int, gh: int, gw: int):
        key = (t, gh, gw)
        if key not in self._tables:
            hd = self.cfg.hidden // self.cfg.heads
            self._tables[key] = (axial_freqs_2d(gh, gw, hd // 2, self.cfg.spatial_max_freq).to(self.device),
                                 temporal_freqs(t, hd).to(self.device))
        return self._tables[key]

    def _half(self, x, cond_act, p: str, angles, temporal: bool):
        """One half-block on x [T, S, D]: adaLN-zero modulated attention, then modulated MLP."""
        c, w = self.cfg, self.w
        d, heads = c.hidden, c.heads
        t, s, _ = x.shape
        mod = _linear(cond_act, w.linear(f"{p}_adaLN_modulation.1", 6 * d, d)).float()[:, None, :]      # [T, 1, 6D]
        sh1, sc1, g1, sh2, sc2, g2 = mod.chunk(6, -1)
        y = (F.layer_norm(x.float(), (d,)) * (1 + sc1) + sh1).to(x.dtype)
        qkv = _linear(y, w.linear(f"{p}_attn.to_qkv", 3 * d, d, bias=False)).view(t, s, 3, heads, d // heads)
        if temporal:      # sequences along time, one per location: [S, heads, T, hd], causal
            q, k, v = (qkv[:, :, i].permute(1, 2, 0, 3) for i in range(3))
            o = _mha(apply_rotary(q, angles), apply_rotary(k, angles), v, causal=True).permute(2, 0, 1, 3)
        else:             # sequences inside a frame: [T, heads, S, hd]
            q, k, v = (qkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))
            o = _mha(apply_rotary(q, angles), apply_rotary(k, angles), v).permute(0, 2, 1, 3)
        x = (x.float() + g1 * _linear(o.reshape(t, s, d), w.linear(f"{p}_attn.to_out", d, d)).float()).to(x.dtype)
        y = (F.layer_norm(x.float(), (d,)) * (1 + sc2) + sh2).to(x.dtype)
        hid = int(d * c.mlp_ratio)
        m = _linear(F.gelu(_linear(y, w.linear(f"{p}_mlp.fc1", hid, d)), approximate="tanh"), w.linear(f"{p}_mlp.fc2", d, hid))
        return (x.float() + g2 * m.float()).to(x.dtype)

    @torch.no_grad()
    def forward(self, latents: torch.Tensor, levels: torch.Tensor, actions: torch.Tensor) -> torch.Tensor:
        """latents [T, C, h, w] (scaled), levels [T] integer noise level per frame, actions [T, 25] ->
        v-prediction [T, C, h, w] fp32. Frame t sees frames <= t only."""
        c, w = self.cfg, self.w
        t, ch, gh, gw = latents.shape
        assert t <= c.max_frames and gh % c.patch == 0 and gw % c.patch == 0
        p = c.patch
        ph, pw = gh // p, gw // p
        x = latents.to(self.device).to(self.dtype).reshape(t, ch, ph, p, pw, p).permute(0, 2, 4, 1, 3, 5).reshape(t, ph * pw, ch * p * p)
        x = _linear(x, w.linear("x_embedder.proj", c.hidden, ch * p * p))
        cond = self._time_embed(levels) + _linear(actions.to(self.device).to(self.dtype), w.linear("external_cond", c.hidden, c.action_dim))
        act = F.silu(cond)
        sp, tm = self._rope(t, ph, pw)
        for i in range(c.depth):
            x = self._half(x, act, f"blocks.{i}.s", sp, False)
            x = self._half(x, act, f"blocks.{i}.t", tm, True)
        d = c.hidden
        sh, sc = _linear(act, w.linear("final_layer.adaLN_modulation.1", 2 * d, d)).float()[:, None, :].chunk(2, -1)
        y = (F.layer_norm(x.float(), (d,)) * (1 + sc) + sh).to(x.dtype)
        out = _linear(y, w.linear("final_layer.linear", p * p * ch, d)).float()
        # token vectors are (row in patch, column in patch, channel)
        return out.reshape(t, ph, pw, p, p, ch).permute(0, 5, 1, 3, 2, 4).reshape(t, ch, gh, gw)


# ---------------------------------------------------------------------------------- sampler
def sigmoid_alphas_cumprod(steps: int, start: float = -3.0, end: float = 3.0, tau: float = 1.0) -> torch.Tensor:
    t = torch.linspace(0, steps, steps + 1, dtype=torch.float64) / steps
    v0, v1 = torch.sigmoid(torch.tensor(start / tau, dtype=torch.float64)), torch.sigmoid(torch.tensor(end / tau, dtype=torch.float64))
    ac = (-torch.sigmoid((t * (end - start) + start) / tau) + v1) / (v1 - v0)
    ac = ac / ac[0]
    betas = (1 - ac[1:] / ac[:-1]).clamp(0, 0.999)
    return torch.cumprod(1 - betas, 0).float()


class OasisWorld:
    """One world: committed latent frames + their actions. ``reset`` with a first picture, then ``step``
    once per action; every step appends one frame and returns it as RGB."""

    def __init__(self, cfg: OasisConfig, dit: OasisDit, vae: OasisVae, seed: int = 0):
        self.cfg, self.dit, self.vae = cfg, dit, vae
        self.ac = sigmoid_alphas_cumprod(cfg.train_steps)
        self.noise_range = torch.linspace(-1, cfg.train_steps - 1, cfg.ddim_steps + 1).long()
        self.seed = seed
        self.frames: list = []          # scaled latents [C, h, w] fp32 on the model's device
        self.actions: list = []         # [25] per frame (zeros for the first)
        self.last_step_levels: list = []

    def reset(self, rgb: torch.Tensor) -> torch.Tensor:
        """rgb [3, H, W] in [0, 1]. Returns the autoencoder's reconstruction of it, [3, H, W] in [0, 1]."""
        z = self.vae.encode(rgb[None] * 2 - 1)[0] * SCALING
        self.frames, self.actions = [z.float()], [torch.zeros(self.cfg.action_dim)]
        return self.decode_frame(0)

    def decode_frame(self, i: int) -> torch.Tensor:
        return (self.vae.decode((self.frames[i] / SCALING)[None])[0] * 0.5 + 0.5).clamp(0, 1)

    @torch.no_grad()
    def step(self, action: torch.Tensor) -> torch.Tensor:
        """Appends the frame that follows ``action`` [25]; returns it as RGB [3, H, W] in [0, 1]."""
        cfg, dev = self.cfg, self.dit.device
        i = len(self.frames)
        g = torch.Generator().manual_seed(self.seed + i)
        noise = torch.randn(self.frames[0].shape, generator=g).clamp(-cfg.noise_abs_max, cfg.noise_abs_max).to(dev)
        self.actions.append(torch.as_tensor(action, dtype=torch.float32).reshape(cfg.action_dim))
        start = max(0, i + 1 - cfg.max_frames)
        ctx = torch.stack(self.frames[start:]) if i > start else noise[None][:0]
        acts = torch.stack(self.actions[start:])
        x = noise
        ac = self.ac.to(dev)
        n_ctx = ctx.shape[0]
        self.last_step_levels = []
        for k in range(cfg.ddim_steps, 0, -1):
            lv, lv_next = int(self.noise_range[k]), int(self.noise_range[k - 1])
            if lv_next < 0:
                lv_next = lv
            levels = torch.tensor([cfg.stabilization_level - 1] * n_ctx + [lv])
            self.last_step_levels.append(levels.tolist())
            v = self.dit.forward(torch.cat([ctx, x[None]]), levels, acts)[-1]
            a_t = ac[lv]
            x0 = a_t.sqrt() * x - (1 - a_t).sqrt() * v
            eps = ((1 / a_t).sqrt() * x - x0) / (1 / a_t - 1).sqrt()
            a_next = torch.ones((), device=dev) if k == 1 else ac[lv_next]
            x = a_next.sqrt() * x0 + (1 - a_next).sqrt() * eps
        self.frames.append(x.float())
        return self.decode_frame(i)
