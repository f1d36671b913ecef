"""Kyutai streaming speech-to-text: a decoder-only language model that reads Mimi codes and writes text,
one text token per 80 ms audio frame.

Step t consumes the SUM of 33 embeddings from one table: the text token written at step t - 1 (the
start token at t = 0) and the 32 Mimi codes of frame t - 1 (at t = 0 the audio start id in every
codebook), the codes offset into their own ranges behind the text vocabulary. The stack is
pre-RMSNorm attention with rotary positions inside a sliding window and a gated SiLU feed-forward
whose first projection holds [gate | up]; ``lm_head`` gives the next text token, chosen greedily.
The text stream is mostly padding ids: a word appears a fixed delay (2.5 s in the released 2.6 B
model) after it was spoken, so audio is right-padded by that delay (+ 1 s) before transcription,
and one second of silence is put in front.

Audio is coded by :class:`~.mimi.Mimi` (``codec_model.*`` weights of the same checkpoint).
Weights by the names of the `transformers` checkpoint. Reference:
src/HartsyInference.Audio/Models/Kyutai/ (KyutaiSttModel, KyutaiSttConfig, MoshiTransformer),
Pipelines/KyutaiSttPipeline.cs.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.nn.functional as F

from .mimi import Mimi, MimiConfig


@dataclass(frozen=True)
class KyutaiSttConfig:
    vocab: int = 4001
    codebook_vocab: int = 2049
    codebooks: int = 32
    hidden: int = 2048
    layers: int = 48
    heads: int = 32
    kv_heads: int = 32
    head_dim: int = 64
    ffn: int = 11264
    window: int = 375
    eps: float = 1e-8
    theta: float = 10000.0
    bos: int = 48000
    pad: int = 3
    audio_bos: int = 2048
    audio_pad: int = 69569
    frame_size: int = 1920

    @staticmethod
    def from_hf(d: dict) -> "KyutaiSttConfig":
        rope = d.get("rope_parameters") or {}
        heads = d.get("num_attention_heads", 32)
        return KyutaiSttConfig(vocab=d.get("vocab_size", 4001), codebook_vocab=d.get("codebook_vocab_size", 2049),
                               codebooks=d.get("num_codebooks", 32), hidden=d.get("hidden_size", 2048), layers=d.get("num_hidden_layers", 48),
                               heads=heads, kv_heads=d.get("num_key_value_heads", heads), head_dim=d.get("head_dim") or d.get("hidden_size", 2048) // heads,
                               ffn=d.get("ffn_dim", 11264), window=d.get("sliding_window", 375), eps=d.get("rms_norm_eps", 1e-8),
                               theta=float(rope.get("rope_theta", d.get("rope_theta", 10000.0))), bos=d.get("bos_token_id", 48000),
                               pad=d.get("pad_token_id", 3), audio_bos=d.get("audio_bos_token_id", 2048),
                               audio_pad=d.get("audio_pad_token_id", 69569), frame_size=d.get("frame_size", 1920))


class KyutaiStt:
    def __init__(self, raw: dict, get: Callable[[str], Optional[torch.Tensor]], device="cpu", dtype: torch.dtype = torch.float32):
        self.cfg = cfg = KyutaiSttConfig.from_hf(raw)
        self.device, self.dtype = torch.device(device), dtype

        def t(n):
            w = get(n)
            if w is None:
                raise KeyError(n)
            return w.to(self.device).to(dtype)

        self.embed = t("model.embed_tokens.embed_tokens.weight")
        self.blocks = []
        for i in range(cfg.layers):
            p = f"model.layers.{i}."
            self.blocks.append({"ln1": t(p + "input_layernorm.weight"), "ln2": t(p + "post_attention_layernorm.weight"),
                                "qkv": torch.cat([t(p + f"self_attn.{n}_proj.linear.weight") for n in "qkv"], 0),
                                "o": t(p + "self_attn.o_proj.linear.weight"), "fc1": t(p + "mlp.fc1.weight"), "fc2": t(p + "mlp.fc2.weight")})
        self.norm, self.lm_head = t("model.norm.weight"), t("lm_head.weight")
        self.codec = Mimi(MimiConfig.from_hf(raw.get("codec_config", {})), get, device, dtype, prefix="codec_model.")
        offsets = torch.arange(cfg.codebooks, device=self.device) * cfg.codebook_vocab + cfg.vocab
        self._offsets = F.pad(offsets, (1, 0))
        self._inv = 1.0 / (cfg.theta ** (torch.arange(0, cfg.head_dim, 2, device=self.device).float() / cfg.head_dim))

    def _rms(self, x, w):
        return (x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + self.cfg.eps) * w.float()).to(x.dtype)

    def step(self, text: torch.Tensor, codes: torch.Tensor, cache: dict) -> torch.Tensor:
        """text [B] + codes [B, codebooks] of one position -> logits over the text vocabulary [B, vocab]."""
        cfg = self.cfg
        ids = torch.cat([text[:, None], codes], 1).to(self.device).long()
        ids = torch.where(ids == cfg.audio_pad, ids, ids + self._offsets)
        x = self.embed[ids].sum(1)[:, None]                                        # [B, 1, H]
        pos = cache["len"]
        ang = (torch.tensor([float(pos)], device=self.device)[:, None] * self._inv[None])
        cos, sin = torch.cat([ang.cos(), ang.cos()], -1).to(x.dtype), torch.cat([ang.sin(), ang.sin()], -1).to(x.dtype)
        half = cfg.head_dim // 2
        rot = lambda u: u * cos + torch.cat([-u[..., half:], u[..., :half]], -1) * sin
        b = x.shape[0]
        nq, nk = cfg.heads * cfg.head_dim, cfg.kv_heads * cfg.head_dim
        for i, blk in enumerate(self.blocks):
            q, k, v = F.linear(self._rms(x, blk["ln1"]), blk["qkv"]).split([nq, nk, nk], -1)
            q = rot(q.view(b, 1, cfg.heads, cfg.head_dim).transpose(1, 2))
            k = rot(k.view(b, 1, cfg.kv_heads, cfg.head_dim).transpose(1, 2))
            v = v.view(b, 1, cfg.kv_heads, cfg.head_dim).transpose(1, 2)
            if cache["k"][i] is not None:
                k, v = torch.cat([cache["k"][i], k], 2)[:, :, -cfg.window:], torch.cat([cache["v"][i], v], 2)[:, :, -cfg.window:]
            cache["k"][i], cache["v"][i] = k, v
            a = F.scaled_dot_product_attention(q, k, v, enable_gqa=cfg.kv_heads != cfg.heads)
            x = x + F.linear(a.transpose(1, 2).reshape(b, 1, nq), blk["o"])
            g, u = F.linear(self._rms(x, blk["ln2"]), blk["fc1"]).chunk(2, -1)
            x = x + F.linear(F.silu(g) * u, blk["fc2"])
        cache["len"] = pos + 1
        return F.linear(self._rms(x[:, 0], self.norm), self.lm_head).float()

    def new_cache(self) -> dict:
        return {"k": [None] * self.cfg.layers, "v": [None] * self.cfg.layers, "len": 0}

    @torch.no_grad()
    def tokens_from_codes(self, codes: torch.Tensor, max_tokens: Optional[int] = None) -> torch.Tensor:
        """codes [codebooks, frames] -> text tokens [frames] (padding ids included), greedy."""
        cfg = self.cfg
        frames = codes.shape[1] if max_tokens is None else min(max_tokens, codes.shape[1])
        cache = self.new_cache()
        text = torch.tensor([cfg.bos], device=self.device)
        audio = torch.full((1, cfg.codebooks), cfg.audio_bos, device=self.device)
        out = []
        for t_ in range(frames):
            text = self.step(text, audio, cache).argmax(-1)
            out.append(int(text))
            audio = codes[:, t_][None].to(self.device)
        return torch.tensor(out, dtype=torch.long)

    @torch.no_grad()
    def transcribe_tokens(self, wave: torch.Tensor, delay_seconds: float = 0.0, silence_prefix_seconds: float = 0.0) -> torch.Tensor:
        """wave [samples] at the codec's rate -> text tokens, one per frame. The delay (+ 1 s) is padded on the right
        so the last words can come out; the prefix is silence in front, as the model saw in training."""
        rate = self.codec.cfg.sampling_rate
        x = wave.to(self.device).float().flatten()
        if silence_prefix_seconds or delay_seconds:
            x = F.pad(x, (int(silence_prefix_seconds * rate), int((delay_seconds + 1.0) * rate) if delay_seconds else 0))
        usable = x.numel() // self.cfg.frame_size * self.cfg.frame_size
        codes = self.codec.encode(x[:usable].reshape(1, 1, -1))[0]
        return self.tokens_from_codes(codes)

    def text_ids(self, tokens: torch.Tensor) -> list[int]:
        """The written tokens without padding / start ids (0 = end of a word's pieces in this vocabulary is kept)."""
        skip = {self.cfg.pad, self.cfg.bos}
        return [int(t) for t in tokens.tolist() if int(t) not in skip]
