"""gpt-oss feed-forward: a biased top-k router over experts whose gate / up columns are interleaved
and whose activation is a clamped, shifted SwiGLU.

    logits  = x @ Wr^T + br                       top-k of the logits, softmax over the k kept values
    gate,up = (x @ Wgu[e] + bgu[e])[..., 0::2], [..., 1::2]
    act     = (clamp(up, -7, 7) + 1) * g * sigmoid(1.702 g),   g = min(gate, 7)
    y      += w_e * (act @ Wd[e] + bd[e])

The experts are held replicated (every tensor-parallel rank computes the same output, so nothing is
reduced); the routed (token, expert) pairs are grouped by expert so each expert's matrices are read
once per call. Reference architecture list: Transformer/GgufConfigFactory.cs (gpt-oss).
"""
from __future__ import annotations

import torch

ALPHA = 1.702
LIMIT = 7.0


def expert_tensor(get, name: str):
    """``[E, in, out]`` expert matrix ``name``: stored as is, or as MXFP4 ``name_blocks``
    uint8 [E, out, in / 32, 16] + ``name_scales`` E8M0 [E, out, in / 32] (the released checkpoints)."""
    t = get(name)
    if t is not None:
        return t
    blocks, scales = get(name + "_blocks"), get(name + "_scales")
    if blocks is None or scales is None:
        raise KeyError(f"missing tensor {name}")
    from ...assets.lowbit import mxfp4_dequantize
    e, rows = blocks.shape[0], blocks.shape[1]
    flat = blocks.reshape(e * rows, -1)
    w = mxfp4_dequantize(flat, scales.reshape(e * rows, -1))
    return w.reshape(e, rows, -1).transpose(1, 2).contiguous().to(torch.bfloat16)


class GptOssMoe:
    def __init__(self, router_w: torch.Tensor, router_b: torch.Tensor, gate_up: torch.Tensor, gate_up_b: torch.Tensor,
                 down: torch.Tensor, down_b: torch.Tensor, top_k: int):
        # gate_up [E, hidden, 2 * ffn] (columns gate0, up0, gate1, up1, ...), down [E, ffn, hidden]
        self.router_w, self.router_b = router_w, router_b
        self.gate_w, self.up_w = gate_up[..., 0::2].contiguous(), gate_up[..., 1::2].contiguous()
        self.gate_b, self.up_b = gate_up_b[..., 0::2].contiguous(), gate_up_b[..., 1::2].contiguous()
        self.down_w, self.down_b = down, down_b
        self.top_k = top_k

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.router_w, self.router_b, self.gate_w, self.up_w,
                                                          self.gate_b, self.up_b, self.down_w, self.down_b))

    def route(self, x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        logits = x.float() @ self.router_w.float().t() + self.router_b.float()
        top, idx = torch.topk(logits, self.top_k, dim=-1)
        return torch.softmax(top, dim=-1), idx

    def __call__(self, x: torch.Tensor, model=None) -> torch.Tensor:
        t, h = x.shape
        w, idx = self.route(x)
        out = torch.zeros(t, h, dtype=torch.float32, device=x.device)
        # group the routed (token, expert) pairs by expert so that each expert's matrices are read once
        flat_e = idx.reshape(-1)
        order = torch.argsort(flat_e, stable=True)
        tok = torch.arange(t, device=x.device).repeat_interleave(self.top_k)[order]
        counts = torch.bincount(flat_e, minlength=self.router_w.shape[0]).tolist()
        wt = w.reshape(-1)[order]
        a = 0
        for e, n in enumerate(counts):
            if n == 0:
                continue
            rows = tok[a:a + n]
            xe = x[rows].to(self.gate_w.dtype)
            gate = ((xe @ self.gate_w[e]).float() + self.gate_b[e].float()).clamp(max=LIMIT)
            up = ((xe @ self.up_w[e]).float() + self.up_b[e].float()).clamp(-LIMIT, LIMIT)
            act = (up + 1.0) * gate * torch.sigmoid(gate * ALPHA)
            ye = (act.to(self.down_w.dtype) @ self.down_w[e]).float() + self.down_b[e].float()
            out.index_add_(0, rows, ye * wt[a:a + n, None])
            a += n
        return out.to(x.dtype)
