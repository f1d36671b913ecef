"""Llama 3.2 Vision (Mllama) text side: the decoder interleaves ordinary llama layers with
cross-attention layers that read the vision tower's output.

A cross-attention layer (tanh gates start at zero, so an untrained layer is the identity):

    a  = o_proj(attn(q_norm(q_proj(norm1(x))), k_norm(k_proj(s)), v_proj(s)))     no rotary, no causal mask
    x  = x + tanh(g_attn) * a
    x  = x + tanh(g_mlp) * row_mask * mlp(norm2(x))

``s`` are the projected vision states of the sequence ([Tv, hidden]); without them (a text-only
prompt) the layer is skipped altogether, which is what the model was trained to do. K / V of the
vision states are computed once per request and reused while the same states tensor is passed.
Reference architecture list: Transformer/GgufConfigFactory.cs (mllama), Multimodal/ (Mllama).
"""
from __future__ import annotations

from typing import Optional

import torch

from ... import ops
from ...ops import reference as R
from ...ops.core import LinearWeight


class CrossLayer:
    def __init__(self, in_norm: torch.Tensor, post_norm: torch.Tensor, q: LinearWeight, k: LinearWeight, v: LinearWeight,
                 o: LinearWeight, q_norm: torch.Tensor, k_norm: torch.Tensor, gate_up: LinearWeight, down: LinearWeight,
                 attn_gate: float, mlp_gate: float, heads: int, kv_heads: int, head_dim: int, eps: float):
        self.in_norm, self.post_norm = in_norm, post_norm
        self.q, self.k, self.v, self.o = q, k, v, o
        self.q_norm, self.k_norm = q_norm, k_norm
        self.gate_up, self.down = gate_up, down
        self.attn_gate, self.mlp_gate = attn_gate, mlp_gate
        self.heads, self.kv_heads, self.d, self.eps = heads, kv_heads, head_dim, eps
        # id(states) -> (states, K, V): K / V of the image sets in flight (the entry holds the states tensor,
        # so its id stays unique while the entry lives)
        self._kv_cache: dict[int, tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = {}
        self.max_cached = 16

    def nbytes(self) -> int:
        return sum(w.nbytes() for w in (self.q, self.k, self.v, self.o, self.gate_up, self.down))

    def _kv(self, states: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        hit = self._kv_cache.get(id(states))
        if hit is None:
            tv = states.shape[0]
            k = ops.linear(states, self.k).reshape(tv * self.kv_heads, self.d)
            k = ops.norm(k, self.k_norm, eps=self.eps)[0].reshape(tv, self.kv_heads, self.d)
            v = ops.linear(states, self.v).reshape(tv, self.kv_heads, self.d)
            if len(self._kv_cache) >= self.max_cached:                    # drop the oldest entry
                self._kv_cache.pop(next(iter(self._kv_cache)))
            hit = self._kv_cache[id(states)] = (states, k, v)
        return hit[1], hit[2]

    def __call__(self, x: torch.Tensor, states: Optional[torch.Tensor], row_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x [T, hidden] (one sequence), states [Tv, hidden] or None, row_mask [T] (0 for text rows
        that precede every image)."""
        if states is None:
            return x
        t = x.shape[0]
        h = ops.norm(x, self.in_norm, eps=self.eps)[0]
        q = ops.linear(h, self.q).reshape(t * self.heads, self.d)
        q = ops.norm(q, self.q_norm, eps=self.eps)[0].reshape(t, self.heads, self.d)
        k, v = self._kv(states)
        a = R.attention(q, k, v, causal=False, scale=self.d ** -0.5).to(x.dtype).reshape(t, self.heads * self.d)
        x = (x.float() + self.attn_gate * ops.linear(a, self.o).float()).to(x.dtype)
        h2 = ops.norm(x, self.post_norm, eps=self.eps)[0]
        act, _ = ops.glu(ops.linear(h2, self.gate_up), "silu")
        f = ops.linear(act, self.down).float()
        if row_mask is not None:
            f = f * row_mask.float()[:, None]
        return (x.float() + self.mlp_gate * f).to(x.dtype)
