"""MusicGen: text -> music. A T5 encoder conditions a decoder language model over the EnCodec
codebooks, and the EnCodec decoder turns the generated codes into audio.

Decoder input at a step is the sum of one embedding per codebook (the tables have one extra row for
the padding / start token) plus a sinusoidal position ([cos | sin] halves); blocks are pre-LayerNorm
self-attention, cross-attention over the projected text states, and a GELU feed-forward, all
without linear biases; one output head per codebook.

Codebook k is delayed by k steps, so frame f of codebook k is produced at step f + k: the id
matrix [K, steps] starts with a padding column, codebook k stays padding until step k, and after
generation row k is read from column k + 1 on. Generation uses classifier-free guidance: the
unconditional branch sees no text (its cross-attention contributes nothing).
Reference: src/HartsyInference.Audio/ (MusicGen pipeline).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.nn.functional as F


@dataclass(frozen=True)
class MusicgenConfig:
    vocab_size: int = 2048           # codes per codebook; id vocab_size is the padding / start token
    hidden: int = 1024
    layers: int = 24
    heads: int = 16
    ffn: int = 4096
    codebooks: int = 4
    scale_embedding: bool = False
    eps: float = 1e-5

    @staticmethod
    def from_hf(d: dict) -> "MusicgenConfig":
        d = d.get("decoder") or d
        return MusicgenConfig(vocab_size=d.get("vocab_size", 2048), hidden=d.get("hidden_size", 1024), layers=d.get("num_hidden_layers", 24),
                              heads=d.get("num_attention_heads", 16), ffn=d.get("ffn_dim", 4096), codebooks=d.get("num_codebooks", 4),
                              scale_embedding=bool(d.get("scale_embedding", False)))


def sinusoid(positions: torch.Tensor, dim: int) -> torch.Tensor:
    half = dim // 2
    freq = torch.exp(torch.arange(half, dtype=torch.float32, device=positions.device) * -(math.log(10000.0) / (half - 1)))
    ang = positions.float()[:, None] * freq[None]
    return torch.cat([ang.cos(), ang.sin()], -1)


def delay_mask(codebooks: int, steps: int) -> torch.Tensor:
    """[K, steps] bool: True where codebook k holds a real token (columns k + 1 .. steps - K + k)."""
    col = torch.arange(steps)[None, :]
    k = torch.arange(codebooks)[:, None]
    return (col > k) & (col <= steps - codebooks + k)


class MusicgenDecoder:
    def __init__(self, cfg: MusicgenConfig, get: Callable[[str], Optional[torch.Tensor]], device="cpu",
                 dtype: torch.dtype = torch.float32, prefix: str = "decoder."):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype

        def t(n):
            w = get(prefix + n)
            if w is None:
                raise KeyError(f"missing tensor {prefix + n}")
            return w.to(dtype).to(self.device)

        self.embed = [t(f"model.decoder.embed_tokens.{k}.weight") for k in range(cfg.codebooks)]
        self.heads = torch.stack([t(f"lm_heads.{k}.weight") for k in range(cfg.codebooks)])          # [K, V, H]
        self.layers = []
        for i in range(cfg.layers):
            p = f"model.decoder.layers.{i}."
            self.layers.append({n: t(p + n) for n in (
                "self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight", "self_attn.out_proj.weight",
                "self_attn_layer_norm.weight", "self_attn_layer_norm.bias",
                "encoder_attn.q_proj.weight", "encoder_attn.k_proj.weight", "encoder_attn.v_proj.weight", "encoder_attn.out_proj.weight",
                "encoder_attn_layer_norm.weight", "encoder_attn_layer_norm.bias",
                "fc1.weight", "fc2.weight", "final_layer_norm.weight", "final_layer_norm.bias")})
        self.ln_w, self.ln_b = t("model.decoder.layer_norm.weight"), t("model.decoder.layer_norm.bias")

    def new_cache(self) -> dict:
        return {"k": [None] * self.cfg.layers, "v": [None] * self.cfg.layers, "ck": [None] * self.cfg.layers,
                "cv": [None] * self.cfg.layers, "length": 0}

    def _heads(self, x: torch.Tensor) -> torch.Tensor:
        return x.reshape(x.shape[0], self.cfg.heads, -1).transpose(0, 1)                             # [heads, T, d]

    @torch.no_grad()
    def forward(self, ids: torch.Tensor, text: Optional[torch.Tensor], cache: dict) -> torch.Tensor:
        """ids [K, T] appended after the steps already in ``cache``; text [S, hidden] (None: no text)
        -> logits [K, T, vocab]."""
        cfg = self.cfg
        ids = ids.to(self.device)
        t = ids.shape[1]
        x = sum(self.embed[k][ids[k]] for k in range(cfg.codebooks))
        if cfg.scale_embedding:
            x = x * math.sqrt(cfg.hidden)
        x = x + sinusoid(torch.arange(cache["length"], cache["length"] + t, device=self.device), cfg.hidden).to(x.dtype)
        ln = lambda u, w, b: F.layer_norm(u.float(), (cfg.hidden,), w.float(), b.float(), cfg.eps).to(u.dtype)
        for i, lw in enumerate(self.layers):
            h = ln(x, lw["self_attn_layer_norm.weight"], lw["self_attn_layer_norm.bias"])
            q = self._heads(F.linear(h, lw["self_attn.q_proj.weight"]))
            k, v = self._heads(F.linear(h, lw["self_attn.k_proj.weight"])), self._heads(F.linear(h, lw["self_attn.v_proj.weight"]))
            if cache["k"][i] is not None:
                k, v = torch.cat([cache["k"][i], k], 1), torch.cat([cache["v"][i], v], 1)
            cache["k"][i], cache["v"][i] = k, v
            past = k.shape[1] - t
            mask = torch.ones(t, k.shape[1], dtype=torch.bool, device=self.device).tril(past)
            a = F.scaled_dot_product_attention(q[None], k[None], v[None], attn_mask=mask)[0]
            x = x + F.linear(a.transpose(0, 1).reshape(t, -1), lw["self_attn.out_proj.weight"])
            if text is not None:
                h = ln(x, lw["encoder_attn_layer_norm.weight"], lw["encoder_attn_layer_norm.bias"])
                if cache["ck"][i] is None:
                    tx = text.to(self.device, x.dtype)
                    cache["ck"][i] = self._heads(F.linear(tx, lw["encoder_attn.k_proj.weight"]))
                    cache["cv"][i] = self._heads(F.linear(tx, lw["encoder_attn.v_proj.weight"]))
                q = self._heads(F.linear(h, lw["encoder_attn.q_proj.weight"]))
                a = F.scaled_dot_product_attention(q[None], cache["ck"][i][None], cache["cv"][i][None])[0]
                x = x + F.linear(a.transpose(0, 1).reshape(t, -1), lw["encoder_attn.out_proj.weight"])
            h = ln(x, lw["final_layer_norm.weight"], lw["final_layer_norm.bias"])
            x = x + F.linear(F.gelu(F.linear(h, lw["fc1.weight"])), lw["fc2.weight"])
        cache["length"] += t
        x = ln(x, self.ln_w, self.ln_b)
        return torch.einsum("th,kvh->ktv", x.float(), self.heads.float())

    @torch.no_grad()
    def generate(self, text: Optional[torch.Tensor], frames: int, guidance: float = 3.0, sample: bool = False, top_k: int = 250,
                 temperature: float = 1.0, seed: int = 0) -> torch.Tensor:
        """-> codes [K, frames]. ``text`` [S, hidden] are the projected text states."""
        cfg = self.cfg
        K, pad = cfg.codebooks, cfg.vocab_size
        steps = frames + K                                   # column 0 is the start token; row k ends k columns later
        valid = delay_mask(K, steps).to(self.device)
        ids = torch.full((K, steps), pad, dtype=torch.long, device=self.device)
        cond, uncond = self.new_cache(), self.new_cache()
        use_cfg = text is not None and guidance != 1.0
        gen = torch.Generator(device="cpu").manual_seed(seed)
        for s in range(steps - 1):
            cur = ids[:, s:s + 1]
            logits = self.forward(cur, text, cond)[:, 0]
            if use_cfg:
                un = self.forward(cur, None, uncond)[:, 0]
                logits = un + (logits - un) * guidance
            if sample:
                logits = logits / max(temperature, 1e-5)
                kth = logits.topk(min(top_k, logits.shape[-1]), -1).values[:, -1:]
                probs = torch.softmax(logits.masked_fill(logits < kth, float("-inf")), -1)
                nxt = torch.multinomial(probs.cpu(), 1, generator=gen)[:, 0].to(self.device)
            else:
                nxt = logits.argmax(-1)
            ids[:, s + 1] = torch.where(valid[:, s + 1], nxt, torch.full_like(nxt, pad))
        return torch.stack([ids[k, k + 1:k + 1 + frames] for k in range(K)])


class Musicgen:
    """Text encoder + projection + decoder LM + EnCodec decoder from one composite checkpoint
    (``text_encoder.*``, ``enc_to_dec_proj.*``, ``decoder.*``, ``audio_encoder.*``)."""

    def __init__(self, raw: dict, get: Callable[[str], Optional[torch.Tensor]], device="cpu", dtype: torch.dtype = torch.float32):
        from ..encoders.t5 import T5Config, T5Encoder
        from .encodec import EncodecConfig, EncodecDecoder
        self.device = torch.device(device)
        tc = raw["text_encoder"]
        t5 = T5Config(vocab_size=tc["vocab_size"], d_model=tc["d_model"], d_kv=tc["d_kv"], d_ff=tc["d_ff"], num_layers=tc["num_layers"],
                      num_heads=tc["num_heads"], num_buckets=tc.get("relative_attention_num_buckets", 32),
                      max_distance=tc.get("relative_attention_max_distance", 128), eps=tc.get("layer_norm_epsilon", 1e-6),
                      gated="gated" in str(tc.get("feed_forward_proj", "relu")))
        self.text = T5Encoder(t5, device, get=lambda n: get("text_encoder." + n))
        self.cfg = MusicgenConfig.from_hf(raw)
        self.decoder = MusicgenDecoder(self.cfg, get, device, dtype)
        w = get("enc_to_dec_proj.weight")
        self.proj_w = None if w is None else w.to(dtype).to(self.device)
        self.proj_b = None if w is None else get("enc_to_dec_proj.bias").to(dtype).to(self.device)
        self.codec = EncodecDecoder(EncodecConfig.from_hf(raw["audio_encoder"]), lambda n: get("audio_encoder." + n), device)
        self.sampling_rate = self.codec.cfg.sampling_rate

    @torch.no_grad()
    def text_states(self, ids: torch.Tensor) -> torch.Tensor:
        h = self.text.encode(ids).to(self.decoder.dtype)
        return h if self.proj_w is None else F.linear(h, self.proj_w, self.proj_b)

    @torch.no_grad()
    def generate(self, ids: torch.Tensor, frames: int, guidance: float = 3.0, sample: bool = False, seed: int = 0) -> torch.Tensor:
        """prompt token ids [L] -> waveform [channels, frames * hop]."""
        codes = self.decoder.generate(self.text_states(ids), frames, guidance=guidance, sample=sample, seed=seed)
        return self.codec.decode(codes[None])[0]
