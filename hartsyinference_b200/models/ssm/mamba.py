"""Mamba (selective state-space) language model.

Block: RMSNorm -> in_proj (x, z) -> causal depthwise conv1d (k = 4) + SiLU -> x_proj (dt, B, C) ->
dt_proj + softplus -> selective scan ``h_t = exp(dt_t A) h_{t-1} + dt_t B_t x_t``,
``y_t = C_t . h_t + D x_t`` -> gate with SiLU(z) -> out_proj, residual. Generation keeps a
constant-size state per sequence: the last k - 1 conv inputs and the [d_inner, d_state] scan state.
Linears run on the tensor-core GEMM, the scan on ``b200_selective_scan`` (one thread per channel,
state in registers); CPU tensors take the plain PyTorch statement.

Reference: src/HartsyInference.LLM/Ssm/ (Mamba model + SsmGenerationPipeline). Weight names follow
Hugging Face ``MambaForCausalLM`` (``backbone.layers.N.mixer.*``).
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
class MambaConfig:
    vocab_size: int = 50280
    d_model: int = 768
    n_layer: int = 24
    d_state: int = 16
    d_conv: int = 4
    expand: int = 2
    dt_rank: int = 0                 # 0 = ceil(d_model / 16)
    rms_eps: float = 1e-5
    eos_token_id: int = 0
    bcdt_rms_eps: float = 0.0        # > 0: weight-free RMS normalisation of dt, B and C after x_proj (FalconMamba)

    @property
    def d_inner(self) -> int:
        return self.expand * self.d_model

    @property
    def rank(self) -> int:
        return self.dt_rank or math.ceil(self.d_model / 16)


def tiny_mamba() -> MambaConfig:
    return MambaConfig(vocab_size=256, d_model=64, n_layer=2, d_state=16)


@dataclass
class MambaState:
    conv: list[torch.Tensor]     # per layer [d_inner, d_conv - 1]: the last inputs of the conv
    ssm: list[torch.Tensor]      # per layer [d_inner, d_state] fp32


@dataclass
class _Layer:
    norm: torch.Tensor
    in_proj: LinearWeight
    conv_w: torch.Tensor         # [d_inner, d_conv]
    conv_b: torch.Tensor
    x_proj: LinearWeight
    dt_proj: LinearWeight        # with bias
    a: torch.Tensor              # -exp(A_log) fp32 [d_inner, d_state]
    d: torch.Tensor              # fp32 [d_inner]
    out_proj: LinearWeight


def selective_scan(x: torch.Tensor, dt: torch.Tensor, a: torch.Tensor, b: torch.Tensor, c: torch.Tensor,
                   d: torch.Tensor, state: torch.Tensor) -> torch.Tensor:
    """x, dt [T, Di]; a [Di, N]; b, c [T, N]; d [Di]; state [Di, N] fp32, updated in place.
    Returns y [T, Di] (dtype of x)."""
    if x.is_cuda:
        return ops.selective_scan(x, dt, a, b, c, d, state)
    xf, dtf, bf, cf = x.float(), dt.float(), b.float(), c.float()
    ys = []
    h = state
    for t in range(x.shape[0]):
        h = torch.exp(dtf[t, :, None] * a) * h + (dtf[t] * xf[t])[:, None] * bf[t][None, :]
        ys.append((h * cf[t][None, :]).sum(-1) + d * xf[t])
    state.copy_(h)
    return torch.stack(ys).to(x.dtype)


class MambaModel:
    def __init__(self, cfg: MambaConfig, device="cpu", get: Optional[Callable[[str], Optional[torch.Tensor]]] = None,
                 seed: int = 0):
        self.cfg, self.device = cfg, torch.device(device)
        g = torch.Generator().manual_seed(seed)
        dt16 = torch.bfloat16

        def t(name, *shape, std=0.02, ones=False):
            v = get(name) if get is not None else None
            if v is None:
                if get is not None:
                    raise KeyError(f"missing tensor {name}")
                v = torch.ones(*shape) if ones else torch.randn(*shape, generator=g) * std
            return v

        dev = self.device
        self.embed = t("backbone.embeddings.weight", cfg.vocab_size, cfg.d_model).to(dt16).to(dev)
        head = get("lm_head.weight") if get is not None else None
        self.lm_head = LinearWeight((head if head is not None else self.embed).to(dt16).to(dev))
        self.norm_f = t("backbone.norm_f.weight", cfg.d_model, ones=True).to(dt16).to(dev)
        self.layers: list[_Layer] = []
        di, n, r = cfg.d_inner, cfg.d_state, cfg.rank
        # the GEMM wants row pitches that are multiples of 16 bytes: pad the dt rank to a multiple
        # of 8 with zero rows (x_proj) / zero columns (dt_proj); the result is unchanged
        self.r_pad = rp = (r + 7) // 8 * 8

        def pad_rows(w, rows):
            return w if w.shape[0] == rows else torch.cat([w, torch.zeros(rows - w.shape[0], w.shape[1], dtype=w.dtype)])

        for i in range(cfg.n_layer):
            p = f"backbone.layers.{i}."
            a_log = t(p + "mixer.A_log", di, n)
            if get is None:
                a_log = torch.log(torch.arange(1, n + 1, dtype=torch.float32))[None].repeat(di, 1)
            dt_b = t(p + "mixer.dt_proj.bias", di)
            self.layers.append(_Layer(
                norm=t(p + "norm.weight", cfg.d_model, ones=True).to(dt16).to(dev),
                in_proj=LinearWeight(t(p + "mixer.in_proj.weight", 2 * di, cfg.d_model).to(dt16).to(dev)),
                conv_w=t(p + "mixer.conv1d.weight", di, 1, cfg.d_conv, std=0.2).reshape(di, cfg.d_conv).float().to(dev),
                conv_b=t(p + "mixer.conv1d.bias", di).float().to(dev),
                x_proj=LinearWeight((lambda w: torch.cat([pad_rows(w[:r], rp), w[r:]]))(
                    t(p + "mixer.x_proj.weight", r + 2 * n, di)).to(dt16).to(dev)),
                dt_proj=LinearWeight(pad_rows(t(p + "mixer.dt_proj.weight", di, r, std=r ** -0.5).t().contiguous(), rp)
                                     .t().contiguous().to(dt16).to(dev), None, dt_b.to(dt16).to(dev)),
                a=(-torch.exp(a_log.float())).contiguous().to(dev),
                d=t(p + "mixer.D", di, ones=True).float().to(dev),
                out_proj=LinearWeight(t(p + "mixer.out_proj.weight", cfg.d_model, di).to(dt16).to(dev))))

    def new_state(self) -> MambaState:
        c = self.cfg
        return MambaState([torch.zeros(c.d_inner, c.d_conv - 1, device=self.device) for _ in self.layers],
                          [torch.zeros(c.d_inner, c.d_state, device=self.device) for _ in self.layers])

    def _mixer(self, lw: _Layer, h: torch.Tensor, conv_state: torch.Tensor, ssm_state: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        di, n, r, k = cfg.d_inner, cfg.d_state, self.r_pad, cfg.d_conv
        xz = ops.linear(h, lw.in_proj)                                  # [T, 2 Di]
        x, z = xz[:, :di], xz[:, di:]
        # causal depthwise conv over [previous k - 1 inputs | x]
        seq = torch.cat([conv_state.t().to(x.dtype), x], 0).float()     # [T + k - 1, Di]
        conv_state.copy_(seq[-(k - 1):].t())
        win = seq.unfold(0, k, 1)                                        # [T, Di, k]
        xc = F.silu((win * lw.conv_w[None]).sum(-1) + lw.conv_b).to(h.dtype)
        dbc = ops.linear(xc.contiguous(), lw.x_proj)                     # [T, r + 2 N]
        dt_in, b_in, c_in = dbc[:, :r], dbc[:, r:r + n], dbc[:, r + n:]
        if cfg.bcdt_rms_eps > 0:
            def rms(u, count):           # the padded dt columns are zero: divide by the real width
                uf = u.float()
                return (uf * torch.rsqrt(uf.pow(2).sum(-1, keepdim=True) / count + cfg.bcdt_rms_eps)).to(u.dtype)
            dt_in, b_in, c_in = rms(dt_in, cfg.rank), rms(b_in, n), rms(c_in, n)
        dt = F.softplus(ops.linear(dt_in.contiguous(), lw.dt_proj).float())
        y = selective_scan(xc.contiguous(), dt.contiguous(), lw.a, b_in.contiguous(), c_in.contiguous(), lw.d, ssm_state)
        y = (y.float() * F.silu(z.float())).to(h.dtype)
        return ops.linear(y.contiguous(), lw.out_proj)

    @torch.no_grad()
    def forward(self, tokens: torch.Tensor, state: MambaState) -> torch.Tensor:
        """tokens [T] appended to the sequence whose state is ``state`` -> hidden states [T, d_model]."""
        x = ops.embedding(tokens.to(self.device).to(torch.int32), self.embed)
        for i, lw in enumerate(self.layers):
            h, _, _ = ops.norm(x, lw.norm, eps=self.cfg.rms_eps)
            x = (x.float() + self._mixer(lw, h, state.conv[i], state.ssm[i]).float()).to(x.dtype)
        out, _, _ = ops.norm(x, self.norm_f, eps=self.cfg.rms_eps)
        return out

    @torch.no_grad()
    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        return ops.linear(hidden, self.lm_head).float()

    @torch.no_grad()
    def generate(self, prompt: list[int], max_tokens: int = 32, stop_at_eos: bool = True) -> list[int]:
        """Greedy generation: one pass over the prompt, then one token per step on the carried state."""
        st = self.new_state()
        h = self.forward(torch.tensor(prompt, dtype=torch.int32), st)
        out = []
        tok = int(self.logits(h[-1:]).argmax(-1))
        for _ in range(max_tokens):
            out.append(tok)
            if stop_at_eos and tok == self.cfg.eos_token_id:
                break
            h = self.forward(torch.tensor([tok], dtype=torch.int32), st)
            tok = int(self.logits(h).argmax(-1))
        return out
