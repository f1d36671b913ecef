"""Wan-2.1-class video DiT over the fused ops, with Ulysses sequence parallelism.

Architecture (T2V-14B: 40 layers, hidden 5120, 40 heads x 128, FFN 13824, 1x2x2 patches, 512 text
tokens of 4096 dims; src/HartsyInference.Diffusion/Models/Denoisers/WanVideoConfig.cs:143-146).
Block op order follows ``WanVideoBlock.Forward`` (DiTBlocks/WanVideoBlock.cs:93: LayerNorm+modulate,
Q/K/V linears :148-150, full-width RMSNorm on q and k :152-153, interleaved 3-D RoPE :171-172,
self-attention :207, gated residual, cross-attention to the text tokens :361, FFN with tanh-GELU
:394-397) and ``WanVideoTransformer.ForwardCore`` (patch embedding, time MLP -> 6-way modulation,
head; WanVideoTransformer.cs:94-223). The 3-D rotary split is h = w = 2 * floor(d / 6),
t = d - h - w (128 -> 44 / 42 / 42; DiTBlocks/WanRope.cs:18-25).

Sequence parallelism (Ulysses): every rank holds S / sp tokens for all token-wise work; around
self-attention the q / k / v activations are exchanged with an all-to-all so that each rank
attends over the full sequence for heads / sp heads, and the output is exchanged back. The
reference's context parallelism instead all-gathers K and V through host memory on two ranks
(src/HartsyInference.Diffusion/Utilities/CpKvExchange.cs:48) and measured slower than one GPU.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch

from ... import config, log, ops
from ...ops import LinearWeight
from ...parallel.comm import Comm, SingleComm
from .common import WeightFactory, rope_tables, silu, timestep_embedding


@dataclass(frozen=True)
class WanConfig:
    in_channels: int = 16
    out_channels: int = 16
    hidden_size: int = 5120
    num_heads: int = 40
    head_dim: int = 128
    ffn_size: int = 13824
    num_layers: int = 40
    text_dim: int = 4096
    text_len: int = 512
    freq_dim: int = 256
    patch: tuple = (1, 2, 2)
    eps: float = 1e-6
    theta: float = 10000.0

    @property
    def patch_dim(self) -> int:
        return self.in_channels * self.patch[0] * self.patch[1] * self.patch[2]

    @property
    def axes_dim(self) -> tuple:
        hw = 2 * (self.head_dim // 6)
        return (self.head_dim - 2 * hw, hw, hw)


WAN_14B = WanConfig()
WAN_1_3B = WanConfig(hidden_size=1536, num_heads=12, ffn_size=8960, num_layers=30)


def tiny_wan(**over) -> WanConfig:
    kw = dict(hidden_size=128, num_heads=4, head_dim=32, ffn_size=256, num_layers=2, text_dim=64, text_len=16, freq_dim=64)
    kw.update(over)
    return WanConfig(**kw)


@dataclass
class _Block:
    modulation: torch.Tensor          # [6, H] learned offsets added to the time projection
    qkv: LinearWeight
    norm_q: torch.Tensor
    norm_k: torch.Tensor
    o: LinearWeight
    norm3_w: torch.Tensor
    norm3_b: torch.Tensor
    cq: LinearWeight
    ckv: LinearWeight
    cnorm_q: torch.Tensor
    cnorm_k: torch.Tensor
    co: LinearWeight
    ffn_in: LinearWeight
    ffn_out: LinearWeight


def patchify(latents: torch.Tensor, patch) -> tuple[torch.Tensor, tuple[int, int, int]]:
    """[C, T, H, W] -> tokens [T' * H' * W', C * pt * ph * pw] (channel-major inside a patch, the
    layout of the patch-embedding convolution's weight) and the token grid."""
    c, t, h, w = latents.shape
    pt, ph, pw = patch
    g = (t // pt, h // ph, w // pw)
    x = latents.reshape(c, g[0], pt, g[1], ph, g[2], pw).permute(1, 3, 5, 0, 2, 4, 6)
    return x.reshape(g[0] * g[1] * g[2], c * pt * ph * pw), g


def unpatchify(tokens: torch.Tensor, grid, patch, channels: int) -> torch.Tensor:
    """Inverse of :func:`patchify` for the head output, whose per-token layout is [pt, ph, pw, C]."""
    pt, ph, pw = patch
    x = tokens.reshape(grid[0], grid[1], grid[2], pt, ph, pw, channels).permute(6, 0, 3, 1, 4, 2, 5)
    return x.reshape(channels, grid[0] * pt, grid[1] * ph, grid[2] * pw)


class WanTransformer:
    def __init__(self, cfg: WanConfig = WAN_14B, device="cpu", sp_comm: Optional[Comm] = None, fp8: bool = False,
                 get: Optional[Callable[[str], Optional[torch.Tensor]]] = None, seed: int = 0):
        self.cfg = cfg
        self.device = torch.device(device)
        self.comm = sp_comm or SingleComm()
        self.sp, self.sp_rank = self.comm.world, self.comm.rank
        # Ulysses (head exchange) needs whole heads per rank; otherwise the tokens stay where they
        # are and every rank gathers all keys / values (the reference's context-parallel exchange,
        # src/HartsyInference.Diffusion/Utilities/CpKvExchange.cs:48, CpSequencePlan.cs:38)
        self.ulysses = cfg.num_heads % self.sp == 0
        self._fused_exchange = {}        # local token count -> FusedUlyssesAttention
        self.exchange_path = "none" if self.sp == 1 else "nccl all-to-all" if self.ulysses else "nccl all-gather of K / V"
        H = cfg.hidden_size
        f = WeightFactory(self.device, fp8, 0, 1, get, seed)
        self.fp8 = fp8 and self.device.type == "cuda"
        self.patch_embedding = f.linear("patch_embedding", H, cfg.patch_dim, allow_fp8=False)
        self.text_in = f.linear("text_embedding.0", H, cfg.text_dim)
        self.text_out = f.linear("text_embedding.2", H, H)
        self.time_in = f.linear("time_embedding.0", H, cfg.freq_dim, allow_fp8=False)
        self.time_out = f.linear("time_embedding.2", H, H)
        self.time_proj = f.linear("time_projection.1", 6 * H, H)
        self.blocks: list[_Block] = []
        for i in range(cfg.num_layers):
            p = f"blocks.{i}."
            q, k, v = (f.linear(p + f"self_attn.{n}", H, H, allow_fp8=False) for n in ("q", "k", "v"))
            ck, cv = (f.linear(p + f"cross_attn.{n}", H, H, allow_fp8=False) for n in ("k", "v"))
            fp = f.fp8 and self.device.type == "cuda"
            self.blocks.append(_Block(
                modulation=f.tensor(p + "modulation", 6, H).reshape(6, H),
                qkv=LinearWeight.from_dense(torch.cat([q.weight, k.weight, v.weight], 0), torch.cat([q.bias, k.bias, v.bias], 0), fp8=fp),
                norm_q=f.tensor(p + "self_attn.norm_q.weight", H, ones=True), norm_k=f.tensor(p + "self_attn.norm_k.weight", H, ones=True),
                o=f.linear(p + "self_attn.o", H, H),
                norm3_w=f.tensor(p + "norm3.weight", H, ones=True), norm3_b=f.tensor(p + "norm3.bias", H, zeros=True),
                cq=f.linear(p + "cross_attn.q", H, H),
                ckv=LinearWeight.from_dense(torch.cat([ck.weight, cv.weight], 0), torch.cat([ck.bias, cv.bias], 0), fp8=fp),
                cnorm_q=f.tensor(p + "cross_attn.norm_q.weight", H, ones=True), cnorm_k=f.tensor(p + "cross_attn.norm_k.weight", H, ones=True),
                co=f.linear(p + "cross_attn.o", H, H),
                ffn_in=f.linear(p + "ffn.0", cfg.ffn_size, H), ffn_out=f.linear(p + "ffn.2", H, cfg.ffn_size)))
        self.head_mod = f.tensor("head.modulation", 2, H).reshape(2, H)
        self.head = f.linear("head.head", cfg.out_channels * cfg.patch[0] * cfg.patch[1] * cfg.patch[2], H)

    def weight_bytes(self) -> int:
        n = 0
        for obj in [self.__dict__] + [b.__dict__ for b in self.blocks]:
            for v in obj.values():
                if isinstance(v, LinearWeight):
                    n += v.nbytes()
        return n

    # ------------------------------------------------------------------------------------
    def encode_text(self, context: torch.Tensor) -> torch.Tensor:
        """[L, text_dim] -> [L, H] (cached per prompt by the pipeline)."""
        return ops.linear(ops.linear(context.to(torch.bfloat16), self.text_in, act="gelu_tanh"), self.text_out)

    def shard_range(self, total_tokens: int) -> tuple[int, int]:
        per = (total_tokens + self.sp - 1) // self.sp
        a = min(total_tokens, self.sp_rank * per)
        return a, min(total_tokens, a + per)

    def _fused(self, s_l: int, heads: int, d: int):
        """The exchange fused into the attention kernels (parallel/ulysses.py) for this shape, or
        None when it does not apply (CPU ranks, head dim other than 128, flag off, no peer access)."""
        if self.device.type != "cuda" or d != 128 or not config.get("fused_ulysses"):
            return None
        if s_l not in self._fused_exchange:
            from ...parallel.ulysses import FusedUlyssesAttention
            try:
                self._fused_exchange[s_l] = FusedUlyssesAttention(self.comm, s_l, heads, self.device)
                self.exchange_path = "peer stores from the quantisation kernel into the attention kernel's operand buffers"
            except Exception as e:      # no peer mapping between these GPUs: keep the collective form
                log.warn(f"[SequenceParallel] fused exchange unavailable ({type(e).__name__}: {e}); using the NCCL collectives")
                self._fused_exchange[s_l] = None
        return self._fused_exchange[s_l]

    def close(self) -> None:
        for f in self._fused_exchange.values():
            if f is not None:
                f.close()
        self._fused_exchange.clear()

    def _self_attention(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        """q, k, v [S_local, heads, D] -> [S_local, heads * D]."""
        if self.sp == 1:
            o = ops.attention(q, k, v)
            return o.reshape(o.shape[0], -1)
        if not self.ulysses:
            fused = self._fused(q.shape[0], q.shape[1], q.shape[2])
            if fused is not None:                                                 # K / V stored into every rank's buffers
                return fused(q.contiguous(), k.contiguous(), v.contiguous())
            kf = self.comm.all_gather(k.contiguous(), dim=0)                      # [S, heads, D]
            vf = self.comm.all_gather(v.contiguous(), dim=0)
            o = ops.attention(q.contiguous(), kf, vf)
            return o.reshape(o.shape[0], -1)
        fused = self._fused(q.shape[0], q.shape[1], q.shape[2])
        if fused is not None:
            return fused(q.contiguous(), k.contiguous(), v.contiguous())
        a2a = self.comm.all_to_all
        qf, kf, vf = (a2a(t, split_dim=1, concat_dim=0) for t in (q, k, v))      # [S, heads / sp, D]
        o = ops.attention(qf.contiguous(), kf.contiguous(), vf.contiguous())
        o = a2a(o, split_dim=0, concat_dim=1)                                    # [S_local, heads, D]
        return o.reshape(o.shape[0], -1)

    def forward(self, latents: torch.Tensor, timestep: torch.Tensor, context: torch.Tensor) -> torch.Tensor:
        """latents [C, T, H, W] (one sample), timestep scalar tensor (0..1000), context [L, H]
        already passed through :meth:`encode_text`. Returns the velocity [C, T, H, W] fp32. With
        sequence parallelism every rank passes the full latents and gets the full result."""
        cfg = self.cfg
        H, D, heads = cfg.hidden_size, cfg.head_dim, cfg.num_heads
        dt = torch.bfloat16
        tokens, grid = patchify(latents.to(self.device), cfg.patch)
        S = tokens.shape[0]
        if self.sp > 1:
            assert S % self.sp == 0, "token count must divide by the sequence-parallel degree"
        a, b = self.shard_range(S)
        x = ops.linear(tokens[a:b].to(dt).contiguous(), self.patch_embedding)
        # rotary tables of the local tokens
        ft, fh, fw = torch.meshgrid(torch.arange(grid[0]), torch.arange(grid[1]), torch.arange(grid[2]), indexing="ij")
        ids = torch.stack([ft, fh, fw], -1).reshape(-1, 3)[a:b].to(self.device)
        cos, sin = rope_tables(ids, cfg.axes_dim, cfg.theta)
        # time conditioning
        te = timestep_embedding(timestep.reshape(1).to(self.device), cfg.freq_dim, flip_sin_to_cos=True).to(dt)
        e = ops.linear(ops.linear(te, self.time_in, act="silu"), self.time_out)              # [1, H]
        e0 = ops.linear(silu(e), self.time_proj).float().reshape(6, H)                       # [6, H]
        S_l = x.shape[0]
        for blk in self.blocks:
            m = (blk.modulation.float() + e0).to(dt).reshape(1, 6 * H).contiguous()
            xn, _, xq = ops.norm(x, None, shift=m[:, 0:H], scale=m[:, H:2 * H], rows_per_batch=S_l, layernorm=True,
                                 eps=cfg.eps, emit_fp8=self.fp8 and blk.qkv.is_fp8, emit_bf16=not (self.fp8 and blk.qkv.is_fp8))
            qkv = ops.linear(xq if xq is not None else xn, blk.qkv)                           # [S_l, 3H]
            qn, _, _ = ops.norm(qkv[:, 0:H].contiguous(), blk.norm_q, eps=cfg.eps)
            kn, _, _ = ops.norm(qkv[:, H:2 * H].contiguous(), blk.norm_k, eps=cfg.eps)
            packed = torch.cat([qn, kn, qkv[:, 2 * H:]], 1)
            q, k, v = ops.dit_qkv(packed, heads, heads, D, cos=cos, sin=sin)
            att = self._self_attention(q, k, v)
            x = ops.linear(att, blk.o, gate=m[0, 2 * H:3 * H].contiguous(), residual=x)
            # cross-attention to the text tokens (no gate, affine LayerNorm)
            xn, _, _ = ops.norm(x, blk.norm3_w, bias=blk.norm3_b, layernorm=True, eps=cfg.eps)
            cq, _, _ = ops.norm(ops.linear(xn, blk.cq), blk.cnorm_q, eps=cfg.eps)
            ckv = ops.linear(context, blk.ckv)
            ck, _, _ = ops.norm(ckv[:, :H].contiguous(), blk.cnorm_k, eps=cfg.eps)
            L = context.shape[0]
            co = ops.attention(cq.reshape(S_l, heads, D), ck.reshape(L, heads, D), ckv[:, H:].reshape(L, heads, D).contiguous())
            x = ops.linear(co.reshape(S_l, H), blk.co, residual=x)
            # feed-forward
            xn, _, xq = ops.norm(x, None, shift=m[:, 3 * H:4 * H], scale=m[:, 4 * H:5 * H], rows_per_batch=S_l,
                                 layernorm=True, eps=cfg.eps, emit_fp8=self.fp8 and blk.ffn_in.is_fp8,
                                 emit_bf16=not (self.fp8 and blk.ffn_in.is_fp8))
            h = ops.linear(xq if xq is not None else xn, blk.ffn_in, act="gelu_tanh")
            x = ops.linear(h, blk.ffn_out, gate=m[0, 5 * H:6 * H].contiguous(), residual=x)
        hm = (self.head_mod.float() + e.float()).to(dt).reshape(1, 2 * H).contiguous()         # shift, scale
        xn, _, _ = ops.norm(x, None, shift=hm[:, 0:H], scale=hm[:, H:2 * H], rows_per_batch=S_l, layernorm=True, eps=cfg.eps)
        out = ops.linear(xn, self.head).float()                                               # [S_l, pt*ph*pw*C]
        if self.sp > 1:
            out = self.comm.all_gather(out, dim=0)
        return unpatchify(out, grid, cfg.patch, cfg.out_channels)
