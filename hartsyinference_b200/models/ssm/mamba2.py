"""Mamba-2 (state-space duality) language model.

Block: RMSNorm -> in_proj (z, xBC, dt) -> causal depthwise conv1d + SiLU over xBC -> split x, B, C
-> ``dt = softplus(dt + dt_bias)`` per head -> scan with one scalar decay per head,
``h_t = exp(dt_t A) h_{t-1} + dt_t B_t x_t``, ``y_t = C_t . h_t + D x_t`` -> RMSNorm(y * SiLU(z)) ->
out_proj, residual. Each head's scalar A and D are broadcast over its channels, so the scan runs on
the same kernel as Mamba-1 (``b200_selective_scan``), once per B / C group.

Reference: src/HartsyInference.LLM/Ssm/ (Mamba2). Weight names follow Hugging Face
``Mamba2ForCausalLM`` (``backbone.layers.N.mixer.*``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.nn.functional as F

from ... import ops
from ...ops import LinearWeight
from .mamba import MambaState, selective_scan


@dataclass(frozen=True)
class Mamba2Config:
    vocab_size: int = 50288
    d_model: int = 768
    n_layer: int = 24
    d_state: int = 128
    d_conv: int = 4
    expand: int = 2
    head_dim: int = 64
    n_groups: int = 1
    rms_eps: float = 1e-5
    dt_min: float = 0.0
    dt_max: float = float("inf")
    eos_token_id: int = 0

    @property
    def d_inner(self) -> int:
        return self.expand * self.d_model

    @property
    def n_heads(self) -> int:
        return self.d_inner // self.head_dim

    @property
    def conv_dim(self) -> int:
        return self.d_inner + 2 * self.n_groups * self.d_state


def tiny_mamba2(**over) -> Mamba2Config:
    base = dict(vocab_size=256, d_model=64, n_layer=2, d_state=16, head_dim=16, n_groups=1)
    base.update(over)
    return Mamba2Config(**base)


def mamba2_from_hf(d: dict) -> Mamba2Config:
    lim = d.get("time_step_limit") or (0.0, float("inf"))
    return Mamba2Config(vocab_size=d["vocab_size"], d_model=d["hidden_size"], n_layer=d["num_hidden_layers"], d_state=d["state_size"],
                        d_conv=d.get("conv_kernel", 4), expand=d.get("expand", 2), head_dim=d["head_dim"], n_groups=d.get("n_groups", 1),
                        rms_eps=d.get("layer_norm_epsilon", 1e-5), dt_min=float(lim[0]), dt_max=float(lim[1]),
                        eos_token_id=d.get("eos_token_id", 0) or 0)


class Mamba2Model:
    def __init__(self, cfg: Mamba2Config, device="cpu", get: Optional[Callable[[str], Optional[torch.Tensor]]] = None, seed: int = 0):
        self.cfg, self.device = cfg, torch.device(device)
        g = torch.Generator().manual_seed(seed)
        bf = torch.bfloat16
        dev = self.device

        def t(name, *shape, std=0.02, ones=False):
            v = get(name) if get is not None else None
            if v is None:
                if get is not None:
                    raise KeyError(f"missing tensor {name}")
                v = torch.ones(*shape) if ones else torch.randn(*shape, generator=g) * std
            return v

        di, n, nh, cd = cfg.d_inner, cfg.d_state, cfg.n_heads, cfg.conv_dim
        self.embed = t("backbone.embeddings.weight", cfg.vocab_size, cfg.d_model).to(bf).to(dev)
        head = get("lm_head.weight") if get is not None else None
        self.lm_head = LinearWeight((head if head is not None else self.embed).to(bf).to(dev))
        self.norm_f = t("backbone.norm_f.weight", cfg.d_model, ones=True).to(bf).to(dev)
        # in_proj rows are [z | xBC | dt]; the output width is padded to a multiple of 8 for the GEMM
        self.proj_out = di + cd + nh
        pad = (-self.proj_out) % 8
        self.layers = []
        for i in range(cfg.n_layer):
            p = f"backbone.layers.{i}."
            w_in = t(p + "mixer.in_proj.weight", self.proj_out, cfg.d_model)
            if pad:
                w_in = torch.cat([w_in, torch.zeros(pad, cfg.d_model, dtype=w_in.dtype)])
            a_log = t(p + "mixer.A_log", nh)
            if get is None:
                a_log = torch.log(torch.arange(1, nh + 1, dtype=torch.float32))
            self.layers.append(dict(
                norm=t(p + "norm.weight", cfg.d_model, ones=True).to(bf).to(dev),
                in_proj=LinearWeight(w_in.to(bf).to(dev)),
                conv_w=t(p + "mixer.conv1d.weight", cd, 1, cfg.d_conv, std=0.2).reshape(cd, cfg.d_conv).float().to(dev),
                conv_b=t(p + "mixer.conv1d.bias", cd).float().to(dev),
                dt_bias=t(p + "mixer.dt_bias", nh).float().to(dev),
                # per-head scalars broadcast to the layout the scan kernel takes: a [Di, N], d [Di]
                a=(-torch.exp(a_log.float())).repeat_interleave(cfg.head_dim)[:, None].expand(di, n).contiguous().to(dev),
                d=t(p + "mixer.D", nh, ones=True).float().repeat_interleave(cfg.head_dim).contiguous().to(dev),
                gate_norm=t(p + "mixer.norm.weight", di, ones=True).float().to(dev),
                out_proj=LinearWeight(t(p + "mixer.out_proj.weight", cfg.d_model, di).to(bf).to(dev))))

    def new_state(self) -> MambaState:
        c = self.cfg
        return MambaState([torch.zeros(c.conv_dim, c.d_conv - 1, device=self.device) for _ in self.layers],
                          [torch.zeros(c.d_inner, c.d_state, device=self.device) for _ in self.layers])

    def _mixer(self, lw: dict, h: torch.Tensor, conv_state: torch.Tensor, ssm_state: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        di, n, nh, cd, k, G = cfg.d_inner, cfg.d_state, cfg.n_heads, cfg.conv_dim, cfg.d_conv, cfg.n_groups
        proj = ops.linear(h, lw["in_proj"])
        z, xbc, dt = proj[:, :di], proj[:, di:di + cd], proj[:, di + cd:di + cd + nh]
        seq = torch.cat([conv_state.t().to(xbc.dtype), xbc], 0).float()
        conv_state.copy_(seq[-(k - 1):].t())
        xbc = F.silu((seq.unfold(0, k, 1) * lw["conv_w"][None]).sum(-1) + lw["conv_b"])        # [T, conv_dim] fp32
        x, b, c = xbc[:, :di], xbc[:, di:di + G * n], xbc[:, di + G * n:]
        dt = F.softplus(dt.float() + lw["dt_bias"]).clamp(cfg.dt_min, cfg.dt_max)
        dt_ch = dt.repeat_interleave(cfg.head_dim, 1).contiguous()                             # [T, Di]
        xs = x.to(h.dtype).contiguous()
        per = di // G
        ys = []
        for gi in range(G):          # heads of one group share B and C
            sl = slice(gi * per, (gi + 1) * per)
            st = ssm_state[sl] if G > 1 else ssm_state
            st_c = st.contiguous()
            ys.append(selective_scan(xs[:, sl].contiguous(), dt_ch[:, sl].contiguous(), lw["a"][sl].contiguous(),
                                     b[:, gi * n:(gi + 1) * n].to(h.dtype).contiguous(), c[:, gi * n:(gi + 1) * n].to(h.dtype).contiguous(),
                                     lw["d"][sl].contiguous(), st_c))
            if G > 1:
                ssm_state[sl] = st_c
        y = torch.cat(ys, 1).float() if G > 1 else ys[0].float()
        y = y * F.silu(z.float())
        y = y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + cfg.rms_eps) * lw["gate_norm"]
        return ops.linear(y.to(h.dtype).contiguous(), lw["out_proj"])

    @torch.no_grad()
    def forward(self, tokens: torch.Tensor, state: MambaState) -> torch.Tensor:
        x = ops.embedding(tokens.to(self.device).to(torch.int32), self.embed)
        for i, lw in enumerate(self.layers):
            h, _, _ = ops.norm(x, lw["norm"], eps=self.cfg.rms_eps)
            x = (x.float() + self._mixer(lw, h, state.conv[i], state.ssm[i]).float()).to(x.dtype)
        return ops.norm(x, self.norm_f, eps=self.cfg.rms_eps)[0]

    @torch.no_grad()
    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        return ops.linear(hidden, self.lm_head).float()

    @torch.no_grad()
    def generate(self, prompt: list[int], max_tokens: int = 32, stop_at_eos: bool = True) -> list[int]:
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
