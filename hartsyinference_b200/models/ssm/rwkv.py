"""RWKV (v4) language model: attention-free blocks with a per-channel exponential-decay recurrence.

Time mixing: each projection reads a learned blend of the current and the previous token's
normalised state ("token shift"); ``wkv_t`` is the decayed, softmax-like average of past values
weighted by ``exp(k)`` with a bonus ``time_first`` for the current token, carried as a numerically
safe (numerator, denominator, running maximum) triple; the output is gated by ``sigmoid(r)``.
Channel mixing: squared-ReLU MLP with the same token shift and a sigmoid gate. Generation needs
five vectors of state per layer, whatever the context length. Projections run on the GEMM path of
``ops.linear``; the recurrence is element-wise.

Reference: src/HartsyInference.LLM/Ssm/ (RWKV family; the reference also carries the v6 / v7
variants, which are not built here). Weight names follow Hugging Face ``RwkvForCausalLM``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.nn.functional as F

from ... import ops
from ...ops import LinearWeight


@dataclass(frozen=True)
class RwkvConfig:
    vocab_size: int = 50277
    hidden: int = 768
    layers: int = 12
    attn_hidden: int = 768
    ffn: int = 3072
    eps: float = 1e-5
    eos_token_id: int = 0


def tiny_rwkv() -> RwkvConfig:
    return RwkvConfig(vocab_size=300, hidden=64, layers=2, attn_hidden=64, ffn=128)


def rwkv_from_hf(d: dict) -> RwkvConfig:
    h = d["hidden_size"]
    return RwkvConfig(vocab_size=d["vocab_size"], hidden=h, layers=d["num_hidden_layers"], attn_hidden=d.get("attention_hidden_size") or h,
                      ffn=d.get("intermediate_size") or 4 * h, eps=d.get("layer_norm_epsilon", 1e-5), eos_token_id=d.get("eos_token_id", 0) or 0)


class RwkvModel:
    def __init__(self, cfg: RwkvConfig, device="cpu", get: Optional[Callable[[str], Optional[torch.Tensor]]] = None, seed: int = 0):
        self.cfg, self.device = cfg, torch.device(device)
        g = torch.Generator().manual_seed(seed)
        bf, dev = torch.bfloat16, self.device
        H, A, Fd = cfg.hidden, cfg.attn_hidden, cfg.ffn

        def t(name, *shape, std=0.02, ones=False, zeros=False):
            v = get(name) if get is not None else None
            if v is None:
                if get is not None:
                    raise KeyError(f"missing tensor {name}")
                v = torch.ones(*shape) if ones else torch.zeros(*shape) if zeros else torch.randn(*shape, generator=g) * std
            return v

        vec = lambda name, n, **kw: t(name, n, **kw).reshape(-1).float().to(dev)
        lin = lambda name, o, i: LinearWeight(t(name, o, i).to(bf).to(dev))
        ln = lambda p: (vec(p + ".weight", H, ones=True), vec(p + ".bias", H, zeros=True))
        self.embed = t("rwkv.embeddings.weight", cfg.vocab_size, H).to(bf).to(dev)
        self.head = lin("head.weight", cfg.vocab_size, H)
        self.ln_out = ln("rwkv.ln_out")
        self.blocks = []
        for i in range(cfg.layers):
            p = f"rwkv.blocks.{i}."
            a, f = p + "attention.", p + "feed_forward."
            self.blocks.append(dict(
                pre_ln=ln(p + "pre_ln") if i == 0 else None, ln1=ln(p + "ln1"), ln2=ln(p + "ln2"),
                decay=-torch.exp(vec(a + "time_decay", A)), first=vec(a + "time_first", A),
                mk=vec(a + "time_mix_key", H, ones=True), mv=vec(a + "time_mix_value", H, ones=True), mr=vec(a + "time_mix_receptance", H, ones=True),
                key=lin(a + "key.weight", A, H), value=lin(a + "value.weight", A, H), recept=lin(a + "receptance.weight", A, H),
                out=lin(a + "output.weight", H, A),
                fmk=vec(f + "time_mix_key", H, ones=True), fmr=vec(f + "time_mix_receptance", H, ones=True),
                fkey=lin(f + "key.weight", Fd, H), frecept=lin(f + "receptance.weight", H, H), fvalue=lin(f + "value.weight", H, Fd)))

    def new_state(self) -> list[dict]:
        c, dev = self.cfg, self.device
        z = lambda n: torch.zeros(n, device=dev)
        return [dict(ax=z(c.hidden), fx=z(c.hidden), num=z(c.attn_hidden), den=z(c.attn_hidden), mx=z(c.attn_hidden) - 1e38)
                for _ in self.blocks]

    def _ln(self, x, wb):
        return F.layer_norm(x.float(), (self.cfg.hidden,), wb[0], wb[1], self.cfg.eps)

    @staticmethod
    def _shift(x: torch.Tensor, prev: torch.Tensor) -> torch.Tensor:
        """[T, H] -> the previous token's row for every position (``prev`` before the first)."""
        return torch.cat([prev[None], x[:-1]], 0)

    def _lin(self, x: torch.Tensor, w: LinearWeight) -> torch.Tensor:
        return ops.linear(x.to(torch.bfloat16).contiguous(), w).float()

    @torch.no_grad()
    def forward(self, tokens: torch.Tensor, state: list[dict]) -> torch.Tensor:
        """tokens [T] appended to the sequence whose state is ``state`` -> hidden states [T, H] (fp32)."""
        x = self.embed[tokens.long().to(self.device)].float()
        for b, st in zip(self.blocks, state):
            if b["pre_ln"] is not None:
                x = self._ln(x, b["pre_ln"])
            h = self._ln(x, b["ln1"])
            prev = self._shift(h, st["ax"])
            st["ax"] = h[-1].clone()
            k = self._lin(h * b["mk"] + prev * (1 - b["mk"]), b["key"])
            v = self._lin(h * b["mv"] + prev * (1 - b["mv"]), b["value"])
            r = torch.sigmoid(self._lin(h * b["mr"] + prev * (1 - b["mr"]), b["recept"]))
            num, den, mx = st["num"], st["den"], st["mx"]
            wkv = torch.empty_like(k)
            for t in range(k.shape[0]):
                kt, vt = k[t], v[t]
                m = torch.maximum(mx, kt + b["first"])
                e1, e2 = torch.exp(mx - m), torch.exp(kt + b["first"] - m)
                wkv[t] = (e1 * num + e2 * vt) / (e1 * den + e2)
                m2 = torch.maximum(mx + b["decay"], kt)
                e1, e2 = torch.exp(mx + b["decay"] - m2), torch.exp(kt - m2)
                num, den, mx = e1 * num + e2 * vt, e1 * den + e2, m2
            st["num"], st["den"], st["mx"] = num, den, mx
            x = x + self._lin(r * wkv, b["out"])
            h = self._ln(x, b["ln2"])
            prev = self._shift(h, st["fx"])
            st["fx"] = h[-1].clone()
            kk = torch.relu(self._lin(h * b["fmk"] + prev * (1 - b["fmk"]), b["fkey"])) ** 2
            rr = torch.sigmoid(self._lin(h * b["fmr"] + prev * (1 - b["fmr"]), b["frecept"]))
            x = x + rr * self._lin(kk, b["fvalue"])
        return self._ln(x, self.ln_out)

    @torch.no_grad()
    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        return self._lin(hidden, self.head)

    @torch.no_grad()
    def generate(self, prompt: list[int], max_tokens: int = 32, stop_at_eos: bool = True) -> list[int]:
        st = self.new_state()
        h = self.forward(torch.tensor(prompt), st)
        out, tok = [], int(self.logits(h[-1:]).argmax(-1))
        for _ in range(max_tokens):
            out.append(tok)
            if stop_at_eos and tok == self.cfg.eos_token_id:
                break
            tok = int(self.logits(self.forward(torch.tensor([tok]), st)).argmax(-1))
        return out
