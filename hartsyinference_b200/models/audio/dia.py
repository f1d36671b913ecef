"""Dia: dialogue text -> speech. A byte-level text encoder conditions a decoder over the nine DAC
codebooks; the codes are decoded to 44.1 kHz audio by the DAC codec.

* encoder: byte embedding, pre-RMSNorm blocks of rotary self-attention (no mask) and a SwiGLU
  feed-forward with a fused [gate | up] projection; attention scores are NOT scaled by
  1 / sqrt(head_dim) anywhere in this model.
* decoder: the input at a step is the sum of the nine codebook embeddings (one table, codebook c
  offset by c x vocab); blocks of causal rotary self-attention (grouped KV heads), cross-attention
  over the encoder states (no positions), SwiGLU; one dense head gives nine x vocab logits.
* delay pattern (0, 8, 9, ..., 15): codebook c of frame f is produced at step f + delay[c]; until
  its delay has passed a codebook's input is the start id.
* sampling: two passes per step, text and all-zero text; ``guided = cond + scale (cond - uncond)``
  selects the top-k candidates and the CONDITIONAL logits are kept for them; only codebook 0 may
  end the utterance (and does so only when the end id is its top logit), the others get the end
  id forced ``delay[c]`` steps later and padding afterwards. The frames before the end are put
  back in step (the delays undone) and decoded.

Weights by the names of the `transformers` checkpoint. Reference:
src/HartsyInference.Audio/Models/Dia/ (DiaModel, DiaEncoder, DiaDecoder, DiaDelayPattern,
DiaSampler), Pipelines/DiaPipeline.cs.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.nn.functional as F


@dataclass(frozen=True)
class DiaStackConfig:
    hidden: int
    layers: int
    heads: int
    kv_heads: int
    head_dim: int
    ffn: int
    eps: float
    theta: float
    vocab: int
    cross_heads: int = 0
    cross_kv_heads: int = 0
    cross_head_dim: int = 0

    @staticmethod
    def from_hf(d: dict) -> "DiaStackConfig":
        rope = d.get("rope_parameters") or {}
        heads = d["num_attention_heads"]
        return DiaStackConfig(hidden=d["hidden_size"], layers=d["num_hidden_layers"], heads=heads, kv_heads=d.get("num_key_value_heads") or heads,
                              head_dim=d.get("head_dim") or d["hidden_size"] // heads, ffn=d["intermediate_size"], eps=d.get("norm_eps", 1e-5),
                              theta=float(rope.get("rope_theta", d.get("rope_theta", 10000.0))), vocab=d["vocab_size"],
                              cross_heads=d.get("cross_num_attention_heads", 0), cross_kv_heads=d.get("cross_num_key_value_heads", 0),
                              cross_head_dim=d.get("cross_head_dim", 0))


def _rms(x, w, eps):
    return (x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


def _rope(pos: torch.Tensor, dim: int, theta: float, dtype):
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2, device=pos.device).float() / dim))
    ang = pos.float()[:, None] * inv[None]
    return torch.cat([ang.cos(), ang.cos()], -1).to(dtype), torch.cat([ang.sin(), ang.sin()], -1).to(dtype)


def _rot(u, cos, sin):
    half = u.shape[-1] // 2
    return u * cos + torch.cat([-u[..., half:], u[..., :half]], -1) * sin


class Dia:
    def __init__(self, raw: dict, get: Callable[[str], Optional[torch.Tensor]], device="cpu", dtype: torch.dtype = torch.float32,
                 codec=None):
        self.device, self.dtype = torch.device(device), dtype
        self.enc_cfg = DiaStackConfig.from_hf(raw["encoder_config"])
        self.dec_cfg = DiaStackConfig.from_hf(raw["decoder_config"])
        dec = raw["decoder_config"]
        self.channels = dec.get("num_channels", 9)
        self.eos, self.pad, self.bos = dec.get("eos_token_id", 1024), dec.get("pad_token_id", 1025), dec.get("bos_token_id", 1026)
        self.delays = list(raw.get("delay_pattern") or [0] + list(range(8, 8 + self.channels - 1)))
        self.codec = codec

        def t(n):
            w = get(n)
            if w is None:
                raise KeyError(n)
            return w.to(self.device).to(dtype)

        lin = lambda p, names: torch.cat([t(f"{p}.{n}.weight") for n in names], 0)
        self.enc_embed = t("model.encoder.embedding.weight")
        self.enc_blocks = []
        for i in range(self.enc_cfg.layers):
            p = f"model.encoder.layers.{i}"
            self.enc_blocks.append({"ln1": t(p + ".pre_sa_norm.weight"), "qkv": lin(p + ".self_attention", ["q_proj", "k_proj", "v_proj"]),
                                    "o": t(p + ".self_attention.o_proj.weight"), "ln2": t(p + ".post_sa_norm.weight"),
                                    "gate_up": t(p + ".mlp.gate_up_proj.weight"), "down": t(p + ".mlp.down_proj.weight")})
        self.enc_norm = t("model.encoder.norm.weight")
        self.dec_embed = t("model.decoder.embeddings.embed.weight")
        self.dec_blocks = []
        for i in range(self.dec_cfg.layers):
            p = f"model.decoder.layers.{i}"
            self.dec_blocks.append({"ln1": t(p + ".pre_sa_norm.weight"), "qkv": lin(p + ".self_attention", ["q_proj", "k_proj", "v_proj"]),
                                    "o": t(p + ".self_attention.o_proj.weight"), "ln_c": t(p + ".pre_ca_norm.weight"),
                                    "cq": t(p + ".cross_attention.q_proj.weight"), "ckv": lin(p + ".cross_attention", ["k_proj", "v_proj"]),
                                    "co": t(p + ".cross_attention.o_proj.weight"), "ln2": t(p + ".pre_mlp_norm.weight"),
                                    "gate_up": t(p + ".mlp.gate_up_proj.weight"), "down": t(p + ".mlp.down_proj.weight")})
        self.dec_norm, self.head = t("model.decoder.norm.weight"), t("logits_dense.weight")
        self._offsets = torch.arange(self.channels, device=self.device) * self.dec_cfg.vocab

    @staticmethod
    def _mlp(x, blk):
        g, u = F.linear(x, blk["gate_up"]).chunk(2, -1)
        return F.linear(u * F.silu(g), blk["down"])

    @torch.no_grad()
    def encode_text(self, ids: torch.Tensor) -> torch.Tensor:
        """ids [B, T] bytes -> states [B, T, H]."""
        cfg = self.enc_cfg
        if ids.numel() and (int(ids.max()) >= cfg.vocab or int(ids.min()) < 0):       # checked on the host: never a bad gather index
            raise ValueError(f"text ids must lie in [0, {cfg.vocab})")
        x = self.enc_embed[ids.to(self.device).long()]
        b, t, _ = x.shape
        cos, sin = _rope(torch.arange(t, device=self.device), cfg.head_dim, cfg.theta, x.dtype)
        nq, nk = cfg.heads * cfg.head_dim, cfg.kv_heads * cfg.head_dim
        for blk in self.enc_blocks:
            q, k, v = F.linear(_rms(x, blk["ln1"], cfg.eps), blk["qkv"]).split([nq, nk, nk], -1)
            q = _rot(q.view(b, t, cfg.heads, -1).transpose(1, 2), cos, sin)
            k = _rot(k.view(b, t, cfg.kv_heads, -1).transpose(1, 2), cos, sin)
            v = v.view(b, t, cfg.kv_heads, -1).transpose(1, 2)
            a = F.scaled_dot_product_attention(q, k, v, scale=1.0, enable_gqa=cfg.kv_heads != cfg.heads)
            x = x + F.linear(a.transpose(1, 2).reshape(b, t, nq), blk["o"])
            x = x + self._mlp(_rms(x, blk["ln2"], cfg.eps), blk)
        return _rms(x, self.enc_norm, cfg.eps)

    def new_cache(self, enc: torch.Tensor) -> dict:
        """Self-attention cache + the cross-attention keys / values of every layer, computed once."""
        cfg = self.dec_cfg
        b, t, _ = enc.shape
        cross = []
        for blk in self.dec_blocks:
            k, v = F.linear(enc, blk["ckv"]).chunk(2, -1)
            cross.append((k.view(b, t, cfg.cross_kv_heads, cfg.cross_head_dim).transpose(1, 2),
                          v.view(b, t, cfg.cross_kv_heads, cfg.cross_head_dim).transpose(1, 2)))
        return {"k": [None] * cfg.layers, "v": [None] * cfg.layers, "len": 0, "cross": cross}

    @torch.no_grad()
    def decode_step(self, codes: torch.Tensor, cache: dict) -> torch.Tensor:
        """codes [B, T, channels] (new positions) -> logits [B, T, channels, vocab] in fp32."""
        cfg = self.dec_cfg
        x = self.dec_embed[codes.to(self.device).long() + self._offsets].sum(2)
        b, t, _ = x.shape
        past = cache["len"]
        cos, sin = _rope(torch.arange(past, past + t, device=self.device), cfg.head_dim, cfg.theta, x.dtype)
        nq, nk = cfg.heads * cfg.head_dim, cfg.kv_heads * cfg.head_dim
        for i, blk in enumerate(self.dec_blocks):
            q, k, v = F.linear(_rms(x, blk["ln1"], cfg.eps), blk["qkv"]).split([nq, nk, nk], -1)
            q = _rot(q.view(b, t, cfg.heads, -1).transpose(1, 2), cos, sin)
            k = _rot(k.view(b, t, cfg.kv_heads, -1).transpose(1, 2), cos, sin)
            v = v.view(b, t, cfg.kv_heads, -1).transpose(1, 2)
            if cache["k"][i] is not None:
                k, v = torch.cat([cache["k"][i], k], 2), torch.cat([cache["v"][i], v], 2)
            cache["k"][i], cache["v"][i] = k, v
            mask = torch.ones(t, past + t, dtype=torch.bool, device=self.device).tril(past) if t > 1 else None
            a = F.scaled_dot_product_attention(q, k, v, attn_mask=mask, scale=1.0, enable_gqa=cfg.kv_heads != cfg.heads)
            x = x + F.linear(a.transpose(1, 2).reshape(b, t, nq), blk["o"])
            cq = F.linear(_rms(x, blk["ln_c"], cfg.eps), blk["cq"]).view(b, t, cfg.cross_heads, cfg.cross_head_dim).transpose(1, 2)
            ck, cv = cache["cross"][i]
            a = F.scaled_dot_product_attention(cq, ck, cv, scale=1.0, enable_gqa=cfg.cross_kv_heads != cfg.cross_heads)
            x = x + F.linear(a.transpose(1, 2).reshape(b, t, -1), blk["co"])
            x = x + self._mlp(_rms(x, blk["ln2"], cfg.eps), blk)
        cache["len"] = past + t
        return F.linear(_rms(x, self.dec_norm, cfg.eps), self.head).float().view(b, t, self.channels, cfg.vocab)

    @torch.no_grad()
    def generate_codes(self, text: torch.Tensor, max_steps: int = 3072, guidance: float = 3.0, top_k: Optional[int] = 45,
                       temperature: float = 1.0, sample: bool = False, seed: int = 0) -> torch.Tensor:
        """text [T] bytes -> codes [channels, frames], delays undone, without the closing frame."""
        c, delays = self.channels, torch.tensor(self.delays, device=self.device)
        text = text.to(self.device).long()[None]
        use_cfg = guidance is not None and guidance != 1.0
        enc = self.encode_text(torch.cat([text, torch.zeros_like(text)], 0) if use_cfg else text)
        cache = self.new_cache(enc)
        gen = torch.Generator().manual_seed(seed)
        rows = [torch.full((c,), self.bos, device=self.device)]
        finished = torch.zeros(c, dtype=torch.bool, device=self.device)
        countdown, ending = delays.clone(), False
        limit = max_steps - max(self.delays) - 1
        while len(rows) < max_steps and not bool(finished.all()):
            step = len(rows) - 1
            inp = torch.where(step <= delays, torch.full_like(rows[-1], self.bos), rows[-1])      # a codebook waits out its delay
            logits = self.decode_step(inp[None, None].expand(2 if use_cfg else 1, 1, c), cache)[:, 0]
            if use_cfg:
                cond = logits[0]
                guided = cond + (cond - logits[1]) * guidance
                if top_k:
                    keep = torch.zeros_like(cond, dtype=torch.bool).scatter(-1, guided.topk(min(top_k, guided.shape[-1]), -1).indices, True)
                    guided = cond.masked_fill(~keep, -math.inf)
                scores = guided
            else:
                scores = logits[0]
            if temperature not in (None, 1.0):
                scores = scores / temperature
            scores[1:, self.eos:] = -math.inf                      # only codebook 0 may end the utterance ...
            scores[0, self.eos + 1:] = -math.inf
            top = scores.argmax(-1)
            ends = top == self.eos                                   # ... and only when the end id is its best candidate
            scores[ends, :self.eos] = -math.inf
            scores[~ends, self.eos] = -math.inf
            ending = ending or bool(scores[0].argmax() == self.eos) or len(rows) == limit
            if ending:
                force = countdown == 0
                scores[force] = -math.inf
                scores[force, self.eos] = 0.0
                countdown = countdown - 1
            if sample:
                if top_k:
                    kth = scores.topk(min(top_k, scores.shape[-1]), -1).values[:, -1:]
                    scores = scores.masked_fill(scores < kth, -math.inf)
                tok = torch.multinomial(F.softmax(scores, -1).cpu(), 1, generator=gen)[:, 0].to(self.device)
            else:
                tok = scores.argmax(-1)
            tok = torch.where(finished, torch.full_like(tok, self.pad), tok)
            finished = finished | (tok == self.eos)
            rows.append(tok)
        seq = torch.stack(rows)                                      # [L, C], delayed
        length = seq.shape[0]
        end = length - int((seq[:, 0] == self.pad).sum()) - 1
        idx = (torch.arange(length, device=self.device)[:, None] + delays[None]).clamp(max=length - 1)
        aligned = seq.gather(0, idx)
        start = int((seq[:, 0] == self.bos).sum())
        return aligned[start:end].t().contiguous()

    @torch.no_grad()
    def generate(self, text: torch.Tensor, **kw) -> torch.Tensor:
        """-> mono wave [samples] at the codec's rate."""
        if self.codec is None:
            raise ValueError("no codec was given: pass the DAC codec that belongs to this checkpoint")
        codes = self.generate_codes(text, **kw)
        if codes.shape[1] == 0:
            return torch.zeros(0)
        return self.codec.decode(codes[None].clamp(0, self.eos - 1))[0, 0].float()
