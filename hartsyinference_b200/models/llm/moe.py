"""Mixture-of-experts feed-forward with expert parallelism.

Layout. Activations are replicated over the ranks of the tensor-parallel group (they come out of
an all-reduce), so expert parallelism needs no token exchange: rank r owns experts
``[r * E/W, (r + 1) * E/W)``, computes their weighted contribution for every token, the shared
expert is column/row-sharded like a dense FFN, and ONE all-reduce sums routed and shared partial
outputs. Routing runs on the device on every rank (deterministic, identical results), so there is
no host round trip per layer and the layer is CUDA-graph capturable.

Per pass of <= 1024 tokens: router GEMM -> ``moe_route`` -> ``moe_dispatch_dynamic`` (device-side
plan: every local expert gets as many blocks of ``cap`` slots as its tokens need) -> grouped
gate_up GEMM over the blocks in use (one launch) -> GLU -> grouped down GEMM -> ``moe_combine``
(fixed order, deterministic).

Reference behaviour: src/HartsyInference.LLM/Transformer/MoeFeedForward.cs (Route:186-233,
RouteGroupLimited:240-312, Forward:88-161 with one device-to-host copy of the router logits and
a per-expert gather / GEMM / scatter-add loop) and src/HartsyInference.LLM/Models/DeepSeekV3Model.cs
for the shared expert and the leading dense layers.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch

from ... import ops
from ...ops import LinearWeight
from ...ops import reference as R
from .config import TransformerConfig

_CHUNK = 1024        # tokens per pass: up to 8 runs of 128 tokens share one read of the expert weights


@dataclass
class MoeWeights:
    router: LinearWeight                       # [E, H] bf16 (never fp8: routing is precision sensitive)
    router_bias: Optional[torch.Tensor]        # [E] fp32 selection bias (DeepSeek-V3 noaux_tc)
    gate_up: LinearWeight                      # stacked [E_local * 2F, H]
    down: LinearWeight                         # stacked [E_local * H, F]
    shared_gate_up: Optional[LinearWeight] = None   # [2 * Fs / W, H]
    shared_down: Optional[LinearWeight] = None      # [H, Fs / W]
    shared_gate: Optional[LinearWeight] = None      # [1, H] sigmoid gate of the shared expert (Qwen2-MoE)


class MoeFeedForward:
    """Callable ``(h [T, H], model) -> [T, H]`` plugged into ``LayerWeights.ffn_module``."""

    def __init__(self, cfg: TransformerConfig, weights: MoeWeights, rank: int = 0, world: int = 1,
                 all_reduce: Optional[Callable[[torch.Tensor], torch.Tensor]] = None):
        moe = cfg.moe
        assert moe is not None and moe.num_experts % world == 0
        self.cfg, self.moe, self.w = cfg, moe, weights
        self.rank, self.world = rank, world
        self.e_local = moe.num_experts // world
        self.e0 = rank * self.e_local
        self.all_reduce = all_reduce
        self.hidden = cfg.hidden_size
        self.ffn = moe.expert_ffn
        self._xs: dict[tuple[int, int], torch.Tensor] = {}     # (capacity, runs) -> dispatch buffer

    def nbytes(self) -> int:
        n = 0
        for lw in (self.w.router, self.w.gate_up, self.w.down, self.w.shared_gate_up, self.w.shared_down,
                   self.w.shared_gate):
            if lw is not None:
                n += lw.nbytes()
        return n

    # ---------------------------------------------------------------------------------- pieces
    def route(self, h: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        m = self.moe
        logits = ops.linear(h, self.w.router)
        if not logits.is_cuda:
            logits = logits.float()
        return ops.moe_route(logits, self.w.router_bias, m.top_k, n_group=m.n_group, topk_group=m.topk_group,
                             sigmoid=m.scoring == "sigmoid", norm_topk=m.norm_topk_prob,
                             scale=m.routed_scaling_factor)

    def _shared(self, h: torch.Tensor) -> Optional[torch.Tensor]:
        w = self.w
        if w.shared_gate_up is None:
            return None
        gu = ops.linear(h, w.shared_gate_up)
        fp8 = w.shared_down.is_fp8 and h.is_cuda
        a, a8 = ops.glu(gu, self.cfg.activation, emit_fp8=fp8, emit_bf16=not fp8)
        y = ops.linear(a8 if a8 is not None else a, w.shared_down)
        if w.shared_gate is not None:
            g = torch.sigmoid(ops.linear(h, w.shared_gate).float())
            y = (y.float() * g).to(y.dtype)
        return y

    def _routed_cpu(self, h: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor, out: torch.Tensor) -> None:
        """fp32 statement of the routed path (tokens grouped per local expert)."""
        n2, f, hd = 2 * self.ffn, self.ffn, self.hidden
        acc = out.float()
        for e in range(self.e_local):
            hit = ids == (self.e0 + e)
            tok = hit.any(dim=1).nonzero().flatten()
            if tok.numel() == 0:
                continue
            wt = (wts * hit).sum(dim=1)[tok]
            gu_w = LinearWeight(self.w.gate_up.weight[e * n2:(e + 1) * n2],
                                None if self.w.gate_up.scale is None else
                                self.w.gate_up.scale[e * (n2 // 128):(e + 1) * (n2 // 128)])
            dn_w = LinearWeight(self.w.down.weight[e * hd:(e + 1) * hd],
                                None if self.w.down.scale is None else
                                self.w.down.scale[e * (hd // 128):(e + 1) * (hd // 128)])
            gu = ops.linear(h[tok], gu_w)
            a, _ = ops.glu(gu, self.cfg.activation)
            y = ops.linear(a, dn_w)
            acc[tok] += wt.unsqueeze(1) * y.float()
        out.copy_(acc.to(out.dtype))

    def _routed_gpu(self, h: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor, out: torch.Tensor,
                    accumulate: bool) -> None:
        y, plan = self._experts_gpu(h, ids)
        ops.moe_combine(y, plan.slot_of, wts, out, accumulate=accumulate)

    def _experts_gpu(self, h: torch.Tensor, ids: torch.Tensor):
        """Dispatch + the two grouped GEMMs of this rank's experts: (outputs by slot, dispatch plan)."""
        t = h.shape[0]
        # variable-size dispatch: every expert gets as many blocks of `cap` slots as its tokens need
        # (device-side plan, no host round trip), so the grouped GEMMs run only over blocks that hold
        # tokens, read each active expert's weights once and use an MMA N of `cap`
        cap = ops.moe_block_capacity(t, self.moe.top_k, self.moe.num_experts)
        max_blocks = (t * self.moe.top_k + cap - 1) // cap + self.e_local
        xs = self._xs.get((cap, max_blocks))
        if xs is None:
            xs = torch.zeros(max_blocks * cap, self.hidden, dtype=torch.bfloat16, device=h.device)
            self._xs[(cap, max_blocks)] = xs
        plan = ops.moe_dispatch_dynamic(h, ids, self.e0, self.e_local, cap, xs)
        gu = ops.grouped_linear_dynamic(xs, self.w.gate_up, self.e_local, plan)
        fp8 = self.w.down.is_fp8
        a, a8 = ops.glu(gu, self.cfg.activation, emit_fp8=fp8, emit_bf16=not fp8, fp8_tile_rows=cap)
        y = ops.grouped_linear_dynamic(a8 if a8 is not None else a, self.w.down, self.e_local, plan)
        return y, plan

    def forward_partial(self, h: torch.Tensor, exchange) -> None:
        """This rank's contribution (its experts + its shard of the shared expert) to every row of ``h``
        [T, H], handed to ``exchange.scatter`` uncombined so that the combine kernel can store each
        row at the rank that owns it (parallel/dp_attention.py). T <= 1024."""
        assert h.shape[0] <= _CHUNK
        ids, wts = self.route(h)
        shared = self._shared(h)
        if h.is_cuda:
            y, plan = self._experts_gpu(h.contiguous(), ids)
            exchange.scatter(y, plan.slot_of, wts, shared, self.moe.top_k)
        else:
            out = shared if shared is not None else torch.zeros_like(h)
            self._routed_cpu(h, ids, wts, out)
            exchange.scatter(None, None, None, out, 0)

    # ---------------------------------------------------------------------------------- forward
    def __call__(self, h: torch.Tensor, model=None) -> torch.Tensor:
        t = h.shape[0]
        outs = []
        for c0 in range(0, t, _CHUNK):
            hc = h[c0:c0 + _CHUNK]
            ids, wts = self.route(hc)
            shared = self._shared(hc)
            out = shared if shared is not None else torch.zeros_like(hc)
            if hc.is_cuda:
                self._routed_gpu(hc.contiguous(), ids, wts, out, accumulate=shared is not None)
            else:
                self._routed_cpu(hc, ids, wts, out)
            outs.append(out)
        y = outs[0] if len(outs) == 1 else torch.cat(outs)
        if self.world > 1 and self.all_reduce is not None:
            y = self.all_reduce(y)
        return y


def moe_reference(h: torch.Tensor, cfg: TransformerConfig, full: dict[str, torch.Tensor]) -> torch.Tensor:
    """Dense fp32 oracle over unsharded weights: ``full`` holds ``router`` [E, H], optional
    ``router_bias`` [E], ``gate_up`` [E, 2F, H], ``down`` [E, H, F], optional ``shared_gate_up``
    [2Fs, H] / ``shared_down`` [H, Fs]."""
    m = cfg.moe
    x = h.float()
    # the router GEMM emits bf16 logits (fp32 accumulation): round the oracle's the same way so
    # that near-ties pick the same experts
    logits = (x @ full["router"].float().t()).to(torch.bfloat16).float()
    ids, wts = R.moe_route(logits, full.get("router_bias"), m.top_k, m.n_group, m.topk_group,
                           m.scoring == "sigmoid", m.norm_topk_prob, m.routed_scaling_factor)
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for j in range(m.top_k):
            e = int(ids[t, j])
            gu = full["gate_up"][e].float() @ x[t]
            a = R.glu(gu.unsqueeze(0), cfg.activation)[0]
            out[t] += wts[t, j] * (full["down"][e].float() @ a)
    if "shared_gate_up" in full:
        gu = x @ full["shared_gate_up"].float().t()
        out += R.glu(gu, cfg.activation) @ full["shared_down"].float().t()
    return out
