"""Building blocks shared by the DiT families: sinusoidal timestep embeddings, N-D rotary tables,
weight construction (bf16 or fp8 block-scaled, optionally sharded for tensor parallelism) and small
helpers over the fused ops."""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch

from ... import ops
from ...ops import LinearWeight


def timestep_embedding(t: torch.Tensor, dim: int, max_period: float = 10000.0, flip_sin_to_cos: bool = True,
                       downscale_freq_shift: float = 0.0) -> torch.Tensor:
    """Sinusoidal embedding of scalar timesteps [B] -> [B, dim] fp32. ``flip_sin_to_cos`` puts the
    cosine half first (Flux: FluxTransformer.cs:947-950)."""
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(half, dtype=torch.float32, device=t.device) /
                      (half - downscale_freq_shift))
    args = t.float()[:, None] * freqs[None]
    emb = torch.cat([torch.sin(args), torch.cos(args)], dim=-1)
    if flip_sin_to_cos:
        emb = torch.cat([emb[:, half:], emb[:, :half]], dim=-1)
    return emb


def rope_tables(ids: torch.Tensor, axes_dim: Sequence[int], theta: float = 10000.0) -> tuple[torch.Tensor, torch.Tensor]:
    """ids [T, n_axes] (positions per axis) -> cos, sin [T, sum(axes_dim) / 2] fp32 for interleaved
    pairs; axis a contributes axes_dim[a] / 2 frequencies theta^(-2i / axes_dim[a])."""
    outs = []
    for a, d in enumerate(axes_dim):
        freqs = theta ** (-torch.arange(0, d, 2, dtype=torch.float64, device=ids.device) / d)
        outs.append(ids[:, a].double()[:, None] * freqs[None])
    ang = torch.cat(outs, dim=-1)
    return ang.cos().float().contiguous(), ang.sin().float().contiguous()


class WeightFactory:
    """Creates ``LinearWeight``s from a checkpoint (``get(name)``) or randomly, with the TP slicing
    convention: ``col`` = output features split across ranks, ``row`` = input features split."""

    def __init__(self, device, fp8: bool, tp_rank: int = 0, tp: int = 1, get=None, seed: int = 0, std: float = 0.02):
        self.device = torch.device(device)
        self.fp8 = fp8
        self.tp_rank, self.tp = tp_rank, tp
        self.get = get
        self.std = std
        self._g = torch.Generator().manual_seed(seed)
        self._seed = seed
        self._big = 0

    def _rand(self, *shape, std=None) -> torch.Tensor:
        n = 1
        for d in shape:
            n *= d
        if self.device.type == "cuda" and n >= (1 << 22) and len(shape) == 2:
            # full-size synthetic models: draw the (unsharded) tensor on the device from a counter-based
            # generator: the same values on every rank, without seconds of host random numbers per tensor
            self._big += 1
            t = torch.empty(*shape, dtype=torch.bfloat16, device=self.device)
            ops.fill_random_(t, self._seed * 1000003 + 7919 * self._big + 1, self.std if std is None else std)
            return t
        return (torch.randn(*shape, generator=self._g) * (self.std if std is None else std)).to(torch.bfloat16)

    def tensor(self, name: str, *shape, ones: bool = False, zeros: bool = False) -> torch.Tensor:
        if self.get is not None:
            t = self.get(name)
            if t is None:
                raise KeyError(name)
            return t.to(torch.bfloat16).to(self.device)
        if ones:
            return torch.ones(*shape, dtype=torch.bfloat16, device=self.device)
        if zeros:
            return torch.zeros(*shape, dtype=torch.bfloat16, device=self.device)
        return self._rand(*shape).to(self.device)

    def linear(self, names: Sequence[str] | str, out_f: int | Sequence[int], in_f: int, bias: bool = True,
               shard: Optional[str] = None, allow_fp8: bool = True, head_dim: int = 0) -> LinearWeight:
        """``names``: one checkpoint prefix or several that are concatenated along the output dim
        (fused qkv). ``out_f`` matches. shard: None | 'col' | 'row'."""
        names = [names] if isinstance(names, str) else list(names)
        outs = [out_f] * len(names) if isinstance(out_f, int) else list(out_f)
        ws, bs = [], []
        for n, o in zip(names, outs):
            if self.get is not None:
                w = self.get(n + ".weight")
                if w is None:
                    raise KeyError(n + ".weight")
                b = self.get(n + ".bias") if bias else None
            else:
                w = self._rand(o, in_f)
                b = self._rand(o) if bias else None
            if shard == "col" and self.tp > 1:
                per = w.shape[0] // self.tp
                w = w[self.tp_rank * per:(self.tp_rank + 1) * per]
                if b is not None:
                    b = b[self.tp_rank * per:(self.tp_rank + 1) * per]
            elif shard == "row" and self.tp > 1:
                per = w.shape[1] // self.tp
                w = w[:, self.tp_rank * per:(self.tp_rank + 1) * per]
                if b is not None and self.tp_rank != 0:
                    b = torch.zeros_like(b)        # the bias is added once, on rank 0's partial sum
            ws.append(w)
            if b is not None:
                bs.append(b)
        w = torch.cat([x.to(self.device) for x in ws], 0).contiguous().to(torch.bfloat16)
        b = torch.cat(bs, 0).to(torch.bfloat16).to(self.device) if bs else None
        return LinearWeight.from_dense(w, b, fp8=self.fp8 and allow_fp8 and w.is_cuda and w.shape[1] % 128 == 0)


def silu(x: torch.Tensor) -> torch.Tensor:
    return torch.nn.functional.silu(x.float()).to(x.dtype)


def modulation(temb_act: torch.Tensor, w: LinearWeight) -> torch.Tensor:
    """AdaLN modulation vectors: linear(silu(temb)) -> [B, k * H] bf16 (``temb_act`` is already SiLU'd)."""
    return ops.linear(temb_act, w)
