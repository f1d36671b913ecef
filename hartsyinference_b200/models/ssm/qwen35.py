"""Qwen3.5 hybrid decoder: gated-DeltaNet (linear attention) layers interleaved with gated
full-attention layers.

Gated DeltaNet layer, per value head with state S [dk, dv]:
    qkv = silu(causal depthwise conv(in_proj_qkv(x)));  q, k L2-normalised, q scaled by dk^-1/2
    g   = -exp(A_log) * softplus(in_proj_a(x) + dt_bias);   beta = sigmoid(in_proj_b(x))
    S  <- S * exp(g);   S <- S + k (x) ((v - S^T k) * beta);   o = S^T q
    y   = out_proj(rmsnorm(o) * w * silu(in_proj_z(x)))
Full-attention layer: q_proj gives a query and an output gate per head; per-head RMSNorm (1 + w) on
q / k, rotary embedding on the first quarter of the head, causal attention, output * sigmoid(gate).
Every norm multiplies by (1 + w). The MoE variant replaces every feed-forward by top-k routed
experts (softmax scores renormalised over the chosen k) plus a shared expert scaled by sigmoid(x . w).

State per sequence: conv tail [conv_dim, k - 1] and S per linear layer, K / V grown per attention
layer. The recurrence runs token by token in tensor ops (the recurrent form; no chunked kernel), so
prompts cost one step per token. The interface is the one the other recurrent models give
(``new_state`` / ``forward`` / ``logits`` / ``generate``), so the text service serves it the same way.
Reference: src/HartsyInference.Core/Ssm/ (Qwen35Model).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Optional

import torch
import torch.nn.functional as F

from ... import ops
from ...ops import reference as R
from ...ops.core import LinearWeight


@dataclass(frozen=True)
class Qwen35Config:
    vocab_size: int = 248320
    hidden: int = 4096
    ffn: int = 12288
    layers: int = 32
    heads: int = 16
    kv_heads: int = 4
    head_dim: int = 256
    lin_k_heads: int = 16
    lin_v_heads: int = 32
    lin_k_dim: int = 128
    lin_v_dim: int = 128
    conv_kernel: int = 4
    layer_types: tuple = ()
    rms_eps: float = 1e-6
    rope_theta: float = 10000000.0
    rotary_factor: float = 0.25
    tie_embeddings: bool = False
    eos_token_id: int = 0
    experts: int = 0                 # > 0: every feed-forward is top-k routed experts + a sigmoid-gated shared expert
    top_k: int = 0
    expert_ffn: int = 0
    shared_ffn: int = 0

    @property
    def rot(self) -> int:
        return int(self.head_dim * self.rotary_factor)


def qwen35_from_hf(d: dict) -> Qwen35Config:
    d = d.get("text_config") or d
    rp = d.get("rope_parameters") or d.get("rope_scaling") or {}
    n = d["num_hidden_layers"]
    types = tuple(d.get("layer_types") or ["full_attention" if (i + 1) % 4 == 0 else "linear_attention" for i in range(n)])
    eos = d.get("eos_token_id", 0)
    return Qwen35Config(vocab_size=d["vocab_size"], hidden=d["hidden_size"], ffn=int(d.get("intermediate_size") or 0), layers=n,
                        heads=d["num_attention_heads"], kv_heads=d.get("num_key_value_heads") or d["num_attention_heads"],
                        head_dim=d.get("head_dim") or d["hidden_size"] // d["num_attention_heads"],
                        lin_k_heads=d.get("linear_num_key_heads", 16), lin_v_heads=d.get("linear_num_value_heads", 32),
                        lin_k_dim=d.get("linear_key_head_dim", 128), lin_v_dim=d.get("linear_value_head_dim", 128),
                        conv_kernel=d.get("linear_conv_kernel_dim", 4), layer_types=types, rms_eps=d.get("rms_norm_eps", 1e-6),
                        rope_theta=float(rp.get("rope_theta") or d.get("rope_theta") or 1e7),
                        rotary_factor=float(rp.get("partial_rotary_factor") or d.get("partial_rotary_factor") or 0.25),
                        tie_embeddings=bool(d.get("tie_word_embeddings", False)),
                        experts=int(d.get("num_experts") or 0), top_k=int(d.get("num_experts_per_tok") or 0),
                        expert_ffn=int(d.get("moe_intermediate_size") or 0),
                        shared_ffn=int(d.get("shared_expert_intermediate_size") or 0),
                        eos_token_id=(eos[0] if isinstance(eos, (list, tuple)) else eos) or 0)


@dataclass
class Qwen35State:
    conv: list = field(default_factory=list)       # per layer: [conv_dim, k - 1] or None
    rec: list = field(default_factory=list)        # per layer: [Hv, dk, dv] fp32 or None
    k: list = field(default_factory=list)          # per layer: [T, Hkv, d] or None
    v: list = field(default_factory=list)
    length: int = 0


def _rms1(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * (1.0 + w.float())).to(x.dtype)


class Qwen35Model:
    def __init__(self, cfg: Qwen35Config, device="cpu", get: Optional[Callable[[str], Optional[torch.Tensor]]] = None,
                 dtype: torch.dtype = torch.bfloat16):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        if get is None:
            raise ValueError("Qwen35Model needs a checkpoint")

        def t(n, dt=dtype):
            w = get(n)
            if w is None:
                raise KeyError(f"missing tensor {n}")
            return w.to(dt).to(self.device)

        lin = lambda n: LinearWeight(t(n).contiguous())
        self.embed = t("model.embed_tokens.weight")
        self.final_norm = t("model.norm.weight")
        head = get("lm_head.weight")
        self.lm_head = LinearWeight(self.embed if (cfg.tie_embeddings or head is None) else head.to(dtype).to(self.device))
        self.layers = []
        for i in range(cfg.layers):
            p = f"model.layers.{i}."
            lw = dict(kind=cfg.layer_types[i], n1=t(p + "input_layernorm.weight"), n2=t(p + "post_attention_layernorm.weight"))
            if cfg.experts > 0:
                m = p + "mlp."
                lw.update(router=t(m + "gate.weight", torch.float32), e_gate_up=t(m + "experts.gate_up_proj"), e_down=t(m + "experts.down_proj"),
                          gate_up=LinearWeight(torch.cat([t(m + "shared_expert.gate_proj.weight"), t(m + "shared_expert.up_proj.weight")]).contiguous()),
                          down=lin(m + "shared_expert.down_proj.weight"), shared_gate=t(m + "shared_expert_gate.weight", torch.float32))
            else:
                lw.update(gate_up=LinearWeight(torch.cat([t(p + "mlp.gate_proj.weight"), t(p + "mlp.up_proj.weight")]).contiguous()),
                          down=lin(p + "mlp.down_proj.weight"))
            if lw["kind"] == "linear_attention":
                a = p + "linear_attn."
                lw.update(qkv=lin(a + "in_proj_qkv.weight"), z=lin(a + "in_proj_z.weight"),
                          ba=LinearWeight(torch.cat([t(a + "in_proj_b.weight"), t(a + "in_proj_a.weight")]).contiguous()),
                          conv=t(a + "conv1d.weight", torch.float32).squeeze(1), dt_bias=t(a + "dt_bias", torch.float32),
                          a_neg=-t(a + "A_log", torch.float32).exp(), norm=t(a + "norm.weight", torch.float32), out=lin(a + "out_proj.weight"))
            else:
                a = p + "self_attn."
                lw.update(q=lin(a + "q_proj.weight"), kv=LinearWeight(torch.cat([t(a + "k_proj.weight"), t(a + "v_proj.weight")]).contiguous()),
                          o=lin(a + "o_proj.weight"), qn=t(a + "q_norm.weight"), kn=t(a + "k_norm.weight"))
            self.layers.append(lw)
        self.inv_freq = (cfg.rope_theta ** (-torch.arange(0, cfg.rot, 2, dtype=torch.float32) / cfg.rot)).to(self.device)

    def new_state(self) -> Qwen35State:
        n = self.cfg.layers
        return Qwen35State(conv=[None] * n, rec=[None] * n, k=[None] * n, v=[None] * n)

    # ------------------------------------------------------------------------------------ layers
    def _delta(self, lw: dict, li: int, h: torch.Tensor, st: Qwen35State) -> torch.Tensor:
        cfg = self.cfg
        t = h.shape[0]
        hk, hv, dk, dv, kk = cfg.lin_k_heads, cfg.lin_v_heads, cfg.lin_k_dim, cfg.lin_v_dim, cfg.conv_kernel
        x = ops.linear(h, lw["qkv"]).float()                                           # [T, 2 Hk dk + Hv dv]
        tail = st.conv[li] if st.conv[li] is not None else torch.zeros(x.shape[1], kk - 1, device=x.device)
        seq = torch.cat([tail.t(), x], 0)
        st.conv[li] = seq[-(kk - 1):].t().contiguous()
        x = F.silu((seq.unfold(0, kk, 1) * lw["conv"][None]).sum(-1))                  # [T, C]
        q, k, v = x.split([hk * dk, hk * dk, hv * dv], -1)
        l2 = lambda u: u * torch.rsqrt(u.pow(2).sum(-1, keepdim=True) + 1e-6)
        q = l2(q.reshape(t, hk, dk)) * dk ** -0.5
        k = l2(k.reshape(t, hk, dk))
        v = v.reshape(t, hv, dv)
        if hv != hk:
            q, k = q.repeat_interleave(hv // hk, 1), k.repeat_interleave(hv // hk, 1)
        ba = ops.linear(h, lw["ba"]).float()
        beta = torch.sigmoid(ba[:, :hv])
        decay = (lw["a_neg"] * F.softplus(ba[:, hv:] + lw["dt_bias"])).exp()          # [T, Hv]
        s = st.rec[li] if st.rec[li] is not None else torch.zeros(hv, dk, dv, device=x.device)
        out = torch.empty(t, hv, dv, device=x.device)
        for i in range(t):
            s = s * decay[i, :, None, None]
            mem = (s * k[i, :, :, None]).sum(1)                                        # [Hv, dv]
            s = s + k[i, :, :, None] * ((v[i] - mem) * beta[i, :, None])[:, None, :]
            out[i] = (s * q[i, :, :, None]).sum(1)
        st.rec[li] = s
        z = ops.linear(h, lw["z"]).float().reshape(t, hv, dv)
        y = out * torch.rsqrt(out.pow(2).mean(-1, keepdim=True) + cfg.rms_eps)
        y = (lw["norm"] * y.to(h.dtype)).float() * F.silu(z)
        return ops.linear(y.reshape(t, hv * dv).to(h.dtype).contiguous(), lw["out"])

    def _attn(self, lw: dict, li: int, h: torch.Tensor, st: Qwen35State, pos: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        t, d, hq, hkv, rot = h.shape[0], cfg.head_dim, cfg.heads, cfg.kv_heads, cfg.rot
        qg = ops.linear(h, lw["q"]).reshape(t, hq, 2 * d)
        q, gate = qg[..., :d], qg[..., d:].reshape(t, hq * d)
        kv = ops.linear(h, lw["kv"])
        k, v = kv[:, :hkv * d].reshape(t, hkv, d), kv[:, hkv * d:].reshape(t, hkv, d)
        q, k = _rms1(q, lw["qn"], cfg.rms_eps), _rms1(k, lw["kn"], cfg.rms_eps)
        ang = pos.float()[:, None] * self.inv_freq[None]
        cos, sin = torch.cat([ang, ang], -1).cos()[:, None], torch.cat([ang, ang], -1).sin()[:, None]

        def rope(u):
            r, keep = u[..., :rot].float(), u[..., rot:]
            rh = torch.cat([-r[..., rot // 2:], r[..., : rot // 2]], -1)
            return torch.cat([(r * cos + rh * sin).to(u.dtype), keep], -1)

        q, k = rope(q), rope(k)
        st.k[li] = k if st.k[li] is None else torch.cat([st.k[li], k], 0)
        st.v[li] = v if st.v[li] is None else torch.cat([st.v[li], v], 0)
        a = R.attention(q, st.k[li], st.v[li], causal=True, scale=d ** -0.5).to(h.dtype).reshape(t, hq * d)
        a = (a.float() * torch.sigmoid(gate.float())).to(h.dtype)
        return ops.linear(a.contiguous(), lw["o"])

    def _ffn(self, lw: dict, h: torch.Tensor) -> torch.Tensor:
        act, _ = ops.glu(ops.linear(h, lw["gate_up"]), "silu")
        y = ops.linear(act, lw["down"])
        if self.cfg.experts <= 0:
            return y
        # shared expert scaled by sigmoid(x . w), plus the top-k experts weighted by their renormalised softmax scores
        out = y.float() * torch.sigmoid(h.float() @ lw["shared_gate"].t())
        probs = torch.softmax(h.float() @ lw["router"].t(), -1)
        top, idx = torch.topk(probs, self.cfg.top_k, -1)
        top = top / top.sum(-1, keepdim=True)
        for e in idx.unique().tolist():
            rows, slot = (idx == e).nonzero(as_tuple=True)
            xe = h[rows]
            gu = xe @ lw["e_gate_up"][e].t()
            f = gu.shape[1] // 2
            ye = (F.silu(gu[:, :f].float()) * gu[:, f:].float()).to(h.dtype) @ lw["e_down"][e].t()
            out.index_add_(0, rows, ye.float() * top[rows, slot][:, None])
        return out.to(h.dtype)

    @torch.no_grad()
    def forward(self, tokens: torch.Tensor, state: Qwen35State) -> torch.Tensor:
        """tokens [T] appended to the sequence held in ``state`` -> final-normed hidden states [T, H]."""
        cfg = self.cfg
        tokens = tokens.to(self.device).long()
        x = self.embed[tokens]
        pos = torch.arange(state.length, state.length + tokens.numel(), device=self.device)
        for li, lw in enumerate(self.layers):
            h = _rms1(x, lw["n1"], cfg.rms_eps)
            a = self._delta(lw, li, h, state) if lw["kind"] == "linear_attention" else self._attn(lw, li, h, state, pos)
            x = (x.float() + a.float()).to(x.dtype)
            h = _rms1(x, lw["n2"], cfg.rms_eps)
            x = (x.float() + self._ffn(lw, h).float()).to(x.dtype)
        state.length += tokens.numel()
        return _rms1(x, self.final_norm, cfg.rms_eps)

    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        return ops.linear(hidden, self.lm_head).float()

    @torch.no_grad()
    def generate(self, prompt: list[int], max_tokens: int = 32, stop_at_eos: bool = True) -> list[int]:
        st = self.new_state()
        h = self.forward(torch.tensor(prompt), st)
        out: list[int] = []
        tok = int(self.logits(h[-1:]).argmax(-1))
        for _ in range(max_tokens):
            out.append(tok)
            if stop_at_eos and tok == self.cfg.eos_token_id:
                break
            tok = int(self.logits(self.forward(torch.tensor([tok]), st)).argmax(-1))
        return out
