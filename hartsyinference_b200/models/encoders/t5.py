"""T5-v1.1 / umT5 encoder (RMS LayerNorm, relative-position attention bias, gated-GELU FFN).
T5-XXL (24 layers, d_model 4096, 64 heads x 64, d_ff 10240) conditions Flux; umT5-XXL (per-layer
position bias) conditions Wan. Reference: src/HartsyInference.Diffusion/Models/TextEncoders/ and
src/HartsyInference.LLM/Seq2Seq/T5Model.cs. Linears run through the tcgen05 GEMM; attention uses
PyTorch SDPA because of the additive bias (the encoder runs once per prompt)."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.nn.functional as F

from ... import ops
from ..dit.common import WeightFactory


@dataclass(frozen=True)
class T5Config:
    vocab_size: int = 32128
    d_model: int = 4096
    num_layers: int = 24
    num_heads: int = 64
    d_kv: int = 64
    d_ff: int = 10240
    num_buckets: int = 32
    max_distance: int = 128
    per_layer_bias: bool = False      # umT5
    eps: float = 1e-6
    gated: bool = True                # False: the original T5 feed-forward, wo(relu(wi(x)))


T5_XXL = T5Config()
UMT5_XXL = T5Config(vocab_size=256384, per_layer_bias=True)


def tiny_t5(**over) -> T5Config:
    kw = dict(vocab_size=128, d_model=64, num_layers=2, num_heads=4, d_kv=16, d_ff=128)
    kw.update(over)
    return T5Config(**kw)


def _relative_buckets(n: int, num_buckets: int, max_distance: int, device) -> torch.Tensor:
    ctx = torch.arange(n, device=device)[:, None]
    mem = torch.arange(n, device=device)[None, :]
    rel = mem - ctx
    nb = num_buckets // 2
    ret = (rel > 0).long() * nb
    rel = rel.abs()
    max_exact = nb // 2
    large = max_exact + (torch.log(rel.float().clamp_min(1) / max_exact) / math.log(max_distance / max_exact) *
                         (nb - max_exact)).long()
    large = large.clamp_max(nb - 1)
    return ret + torch.where(rel < max_exact, rel, large)


class T5Encoder:
    def __init__(self, cfg: T5Config = T5_XXL, device="cpu", fp8: bool = False,
                 get: Optional[Callable[[str], Optional[torch.Tensor]]] = None, seed: int = 0):
        self.cfg, self.device = cfg, torch.device(device)
        f = WeightFactory(self.device, fp8, get=get, seed=seed)
        inner = cfg.num_heads * cfg.d_kv
        self.embed = f.tensor("shared.weight", cfg.vocab_size, cfg.d_model)
        self.layers = []
        for i in range(cfg.num_layers):
            p = f"encoder.block.{i}.layer."
            lw = dict(
                ln1=f.tensor(p + "0.layer_norm.weight", cfg.d_model, ones=True),
                qkv=ops.LinearWeight.from_dense(torch.cat([f.linear(p + f"0.SelfAttention.{n}", inner, cfg.d_model, bias=False, allow_fp8=False).weight
                                                           for n in ("q", "k", "v")], 0), fp8=f.fp8 and self.device.type == "cuda"),
                o=f.linear(p + "0.SelfAttention.o", cfg.d_model, inner, bias=False),
                ln2=f.tensor(p + "1.layer_norm.weight", cfg.d_model, ones=True),
                wi=(ops.LinearWeight.from_dense(torch.cat([f.linear(p + "1.DenseReluDense.wi_0", cfg.d_ff, cfg.d_model, bias=False, allow_fp8=False).weight,
                                                           f.linear(p + "1.DenseReluDense.wi_1", cfg.d_ff, cfg.d_model, bias=False, allow_fp8=False).weight], 0),
                                                fp8=f.fp8 and self.device.type == "cuda") if cfg.gated else
                    f.linear(p + "1.DenseReluDense.wi", cfg.d_ff, cfg.d_model, bias=False)),
                wo=f.linear(p + "1.DenseReluDense.wo", cfg.d_model, cfg.d_ff, bias=False))
            if i == 0 or cfg.per_layer_bias:
                lw["rel"] = f.tensor(p + "0.SelfAttention.relative_attention_bias.weight", cfg.num_buckets, cfg.num_heads)
            self.layers.append(lw)
        self.final_ln = f.tensor("encoder.final_layer_norm.weight", cfg.d_model, ones=True)

    @torch.no_grad()
    def encode(self, ids: torch.Tensor, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        """ids [L] int -> [L, d_model] bf16. ``mask`` [L] bool marks real tokens (padding keys are ignored)."""
        cfg = self.cfg
        L = ids.shape[0]
        x = self.embed[ids.long().to(self.device)]
        buckets = _relative_buckets(L, cfg.num_buckets, cfg.max_distance, self.device)
        bias = None
        for lw in self.layers:
            if "rel" in lw:
                bias = lw["rel"].float()[buckets].permute(2, 0, 1)            # [heads, L, L]
                if mask is not None:
                    bias = bias.masked_fill(~mask.to(self.device)[None, None, :], float("-inf"))
            h, _, _ = ops.norm(x, lw["ln1"], eps=cfg.eps)
            qkv = ops.linear(h, lw["qkv"]).float().reshape(L, 3, cfg.num_heads, cfg.d_kv)
            q, k, v = (qkv[:, i].transpose(0, 1) for i in range(3))           # [heads, L, d]
            att = F.scaled_dot_product_attention(q[None], k[None], v[None], attn_mask=bias[None], scale=1.0)[0]
            att = att.transpose(0, 1).reshape(L, -1).to(torch.bfloat16)
            x = ops.linear(att, lw["o"], residual=x)
            h, _, _ = ops.norm(x, lw["ln2"], eps=cfg.eps)
            if cfg.gated:
                g, _ = ops.glu(ops.linear(h, lw["wi"]), "gelu_tanh")
            else:
                g = torch.relu(ops.linear(h, lw["wi"]))
            x = ops.linear(g, lw["wo"], residual=x)
        out, _, _ = ops.norm(x, self.final_ln, eps=cfg.eps)
        return out


def _causal_buckets(q_pos: torch.Tensor, k_pos: torch.Tensor, num_buckets: int, max_distance: int) -> torch.Tensor:
    """Decoder (unidirectional) relative-position buckets: only how far back a key lies counts."""
    rel = (q_pos[:, None] - k_pos[None, :]).clamp_min(0)
    max_exact = num_buckets // 2
    large = max_exact + (torch.log(rel.float().clamp_min(1) / max_exact) / math.log(max_distance / max_exact) *
                         (num_buckets - max_exact)).long()
    return torch.where(rel < max_exact, rel, large.clamp_max(num_buckets - 1))


class T5Seq2Seq:
    """Encoder-decoder T5 (v1.1 / Flan layout: gated-GELU feed-forward, separate ``lm_head``) with
    greedy generation: the decoder adds causal self-attention with its own relative-position bias and
    a key / value cache, and cross-attention over the encoder states (projected once per input).

    Reference: src/HartsyInference.LLM/T5Model.cs (``DecodeLogits``, ``Generate``). Tensor names follow
    Hugging Face ``T5ForConditionalGeneration``."""

    def __init__(self, cfg: T5Config, device="cpu", get: Optional[Callable[[str], Optional[torch.Tensor]]] = None, seed: int = 0,
                 decoder_layers: Optional[int] = None, decoder_start_id: int = 0, eos_id: int = 1):
        self.cfg, self.device = cfg, torch.device(device)
        self.encoder = T5Encoder(cfg, device, get=get, seed=seed)
        self.start_id, self.eos_id = decoder_start_id, eos_id
        f = WeightFactory(self.device, False, get=get, seed=seed + 5)
        inner, D = cfg.num_heads * cfg.d_kv, cfg.d_model
        lin = lambda name, o, i: f.linear(name, o, i, bias=False, allow_fp8=False)
        self.layers = []
        for i in range(decoder_layers or cfg.num_layers):
            p = f"decoder.block.{i}.layer."
            lw = dict(ln1=f.tensor(p + "0.layer_norm.weight", D, ones=True),
                      q=lin(p + "0.SelfAttention.q", inner, D), k=lin(p + "0.SelfAttention.k", inner, D),
                      v=lin(p + "0.SelfAttention.v", inner, D), o=lin(p + "0.SelfAttention.o", D, inner),
                      lnx=f.tensor(p + "1.layer_norm.weight", D, ones=True),
                      xq=lin(p + "1.EncDecAttention.q", inner, D), xk=lin(p + "1.EncDecAttention.k", inner, D),
                      xv=lin(p + "1.EncDecAttention.v", inner, D), xo=lin(p + "1.EncDecAttention.o", D, inner),
                      ln2=f.tensor(p + "2.layer_norm.weight", D, ones=True),
                      wi0=lin(p + "2.DenseReluDense.wi_0", cfg.d_ff, D), wi1=lin(p + "2.DenseReluDense.wi_1", cfg.d_ff, D),
                      wo=lin(p + "2.DenseReluDense.wo", D, cfg.d_ff))
            if i == 0:
                lw["rel"] = f.tensor(p + "0.SelfAttention.relative_attention_bias.weight", cfg.num_buckets, cfg.num_heads)
            self.layers.append(lw)
        self.final_ln = f.tensor("decoder.final_layer_norm.weight", D, ones=True)
        head = get("lm_head.weight") if get is not None else None
        self.tied = head is None
        self.head = ops.LinearWeight((head if head is not None else self.encoder.embed).to(torch.bfloat16).to(self.device))

    def _heads(self, x: torch.Tensor) -> torch.Tensor:
        return x.float().reshape(x.shape[0], self.cfg.num_heads, self.cfg.d_kv).transpose(0, 1)

    @torch.no_grad()
    def start(self, enc: torch.Tensor) -> dict:
        cross = [(self._heads(ops.linear(enc, lw["xk"])), self._heads(ops.linear(enc, lw["xv"]))) for lw in self.layers]
        return dict(cross=cross, k=[None] * len(self.layers), v=[None] * len(self.layers), pos=0)

    @torch.no_grad()
    def decode(self, st: dict, tokens: torch.Tensor) -> torch.Tensor:
        """tokens [n] at positions st['pos'].. -> logits [n, vocab] (fp32); the caches grow by n."""
        cfg = self.cfg
        n, p0 = tokens.numel(), st["pos"]
        x = self.encoder.embed[tokens.long().to(self.device)]
        qpos = torch.arange(p0, p0 + n, device=self.device)
        kpos = torch.arange(0, p0 + n, device=self.device)
        buckets = _causal_buckets(qpos, kpos, cfg.num_buckets, cfg.max_distance)
        bias = self.layers[0]["rel"].float()[buckets].permute(2, 0, 1)                  # [heads, n, p0 + n]
        bias = bias.masked_fill(kpos[None, None, :] > qpos[None, :, None], float("-inf"))
        for i, lw in enumerate(self.layers):
            h, _, _ = ops.norm(x, lw["ln1"], eps=cfg.eps)
            q, k, v = self._heads(ops.linear(h, lw["q"])), self._heads(ops.linear(h, lw["k"])), self._heads(ops.linear(h, lw["v"]))
            st["k"][i] = k if st["k"][i] is None else torch.cat([st["k"][i], k], 1)
            st["v"][i] = v if st["v"][i] is None else torch.cat([st["v"][i], v], 1)
            a = F.scaled_dot_product_attention(q[None], st["k"][i][None], st["v"][i][None], attn_mask=bias[None], scale=1.0)[0]
            x = ops.linear(a.transpose(0, 1).reshape(n, -1).to(torch.bfloat16), lw["o"], residual=x)
            h, _, _ = ops.norm(x, lw["lnx"], eps=cfg.eps)
            ck, cv = st["cross"][i]
            a = F.scaled_dot_product_attention(self._heads(ops.linear(h, lw["xq"]))[None], ck[None], cv[None], scale=1.0)[0]
            x = ops.linear(a.transpose(0, 1).reshape(n, -1).to(torch.bfloat16), lw["xo"], residual=x)
            h, _, _ = ops.norm(x, lw["ln2"], eps=cfg.eps)
            g = (F.gelu(ops.linear(h, lw["wi0"]).float(), approximate="tanh") * ops.linear(h, lw["wi1"]).float()).to(torch.bfloat16)
            x = ops.linear(g, lw["wo"], residual=x)
        st["pos"] = p0 + n
        out, _, _ = ops.norm(x, self.final_ln, eps=cfg.eps)
        if self.tied:            # tied embeddings are rescaled before the output projection
            out = (out.float() * cfg.d_model ** -0.5).to(out.dtype)
        return ops.linear(out, self.head).float()

    @torch.no_grad()
    def generate(self, input_ids, max_new: int = 64) -> list[int]:
        enc = self.encoder.encode(torch.as_tensor(input_ids))
        st = self.start(enc)
        tok, out = self.start_id, []
        for _ in range(max_new):
            tok = int(self.decode(st, torch.tensor([tok]))[-1].argmax())
            if tok == self.eos_id:
                break
            out.append(tok)
        return out
