"""CSM (conversational speech model): text + audio context -> Mimi codes -> speech.

Two Llama-style decoders (RMSNorm, rotary attention with grouped KV heads, SwiGLU):

* the *backbone* reads one embedding per position: a text token's embedding, or for an audio frame
  the SUM of the embeddings of its 32 codebook entries (one table of 32 x vocab rows, codebook k
  offset by k x vocab; an all-``codebook_eos`` frame closes an utterance). Its last hidden state,
  through ``lm_head``, gives codebook 0 of the next frame.
* the *depth decoder* then fills in codebooks 1..31 of that frame: position 0 is the backbone's
  hidden state, position j >= 1 the embedding of codebook j - 1's token (same offset table, tied
  to the backbone's when ``tie_codebooks_embeddings``), both projected from the backbone width to
  its own; position j is read out through head j - 1 of a [31, hidden, vocab] weight.

The frame goes back into the backbone as the next input; a frame whose entries are all the
end-of-audio id stops generation, and the frames before it are decoded by Mimi (24 kHz).
Context audio is encoded with Mimi and placed on the ``audio_token_id`` positions of the prompt.
Weights by the names of the `transformers` checkpoint. Reference:
src/HartsyInference.Audio/Models/Csm/ (CsmModel, CsmConfig, CsmWeightRemap), Pipelines/CsmPipeline.cs.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.nn.functional as F

from ..llm.config import RopeScaling
from ..llm.transformer import build_inv_freq
from .mimi import Mimi, MimiConfig


@dataclass(frozen=True)
class CsmDecoderConfig:
    hidden: int
    ffn: int
    layers: int
    heads: int
    kv_heads: int
    head_dim: int
    eps: float
    theta: float
    scaling: RopeScaling

    @staticmethod
    def from_hf(d: dict) -> "CsmDecoderConfig":
        rope = d.get("rope_parameters") or d.get("rope_scaling") or {}
        kind = rope.get("rope_type", rope.get("type", "default"))
        scaling = RopeScaling(kind="llama3", factor=float(rope.get("factor", 1.0)), low_freq_factor=float(rope.get("low_freq_factor", 1.0)),
                              high_freq_factor=float(rope.get("high_freq_factor", 4.0)),
                              original_max_position=int(rope.get("original_max_position_embeddings", 8192))) if kind == "llama3" else RopeScaling()
        heads = d["num_attention_heads"]
        return CsmDecoderConfig(hidden=d["hidden_size"], ffn=d["intermediate_size"], layers=d["num_hidden_layers"], heads=heads,
                                kv_heads=d.get("num_key_value_heads", heads), head_dim=d.get("head_dim") or d["hidden_size"] // heads,
                                eps=d.get("rms_norm_eps", 1e-5), theta=float(rope.get("rope_theta", d.get("rope_theta", 500000.0))),
                                scaling=scaling)


def _rms(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return (x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


class _Decoder:
    """Llama-style stack over ready embeddings, with a growing KV cache."""

    def __init__(self, cfg: CsmDecoderConfig, t: Callable, prefix: str):
        self.cfg = cfg
        self.blocks = []
        for i in range(cfg.layers):
            p = f"{prefix}layers.{i}."
            self.blocks.append({
                "ln1": t(p + "input_layernorm.weight"), "ln2": t(p + "post_attention_layernorm.weight"),
                "qkv": torch.cat([t(p + f"self_attn.{n}_proj.weight") for n in "qkv"], 0), "o": t(p + "self_attn.o_proj.weight"),
                "gate_up": torch.cat([t(p + "mlp.gate_proj.weight"), t(p + "mlp.up_proj.weight")], 0), "down": t(p + "mlp.down_proj.weight")})
        self.norm = t(prefix + "norm.weight")
        self.inv_freq = None

    def new_cache(self) -> dict:
        return {"k": [None] * self.cfg.layers, "v": [None] * self.cfg.layers, "len": 0}

    def __call__(self, x: torch.Tensor, cache: dict) -> torch.Tensor:
        cfg = self.cfg
        b, t, _ = x.shape
        if self.inv_freq is None:
            self.inv_freq, _ = build_inv_freq(cfg.head_dim, cfg.theta, cfg.scaling, x.device)
        past = cache["len"]
        ang = torch.arange(past, past + t, device=x.device).float()[:, None] * self.inv_freq[None]
        cos, sin = torch.cat([ang.cos(), ang.cos()], -1).to(x.dtype), torch.cat([ang.sin(), ang.sin()], -1).to(x.dtype)
        half = cfg.head_dim // 2
        rot = lambda u: u * cos + torch.cat([-u[..., half:], u[..., :half]], -1) * sin
        nq, nk = cfg.heads * cfg.head_dim, cfg.kv_heads * cfg.head_dim
        for i, blk in enumerate(self.blocks):
            q, k, v = F.linear(_rms(x, blk["ln1"], cfg.eps), blk["qkv"]).split([nq, nk, nk], -1)
            q = rot(q.view(b, t, cfg.heads, cfg.head_dim).transpose(1, 2))
            k = rot(k.view(b, t, cfg.kv_heads, cfg.head_dim).transpose(1, 2))
            v = v.view(b, t, cfg.kv_heads, cfg.head_dim).transpose(1, 2)
            if cache["k"][i] is not None:
                k, v = torch.cat([cache["k"][i], k], 2), torch.cat([cache["v"][i], v], 2)
            cache["k"][i], cache["v"][i] = k, v
            if t > 1 and past:
                mask = torch.ones(t, past + t, dtype=torch.bool, device=x.device).tril(past)
                a = F.scaled_dot_product_attention(q, k, v, attn_mask=mask, enable_gqa=True)
            else:
                a = F.scaled_dot_product_attention(q, k, v, is_causal=t > 1, enable_gqa=True)
            x = x + F.linear(a.transpose(1, 2).reshape(b, t, nq), blk["o"])
            g, u = F.linear(_rms(x, blk["ln2"], cfg.eps), blk["gate_up"]).chunk(2, -1)
            x = x + F.linear(F.silu(g) * u, blk["down"])
        cache["len"] = past + t
        return _rms(x, self.norm, cfg.eps)


class Csm:
    def __init__(self, raw: dict, get: Callable[[str], Optional[torch.Tensor]], device="cpu", dtype: torch.dtype = torch.float32):
        self.device, self.dtype = torch.device(device), dtype
        self.codebooks = raw.get("num_codebooks", 32)
        self.vocab = raw.get("vocab_size", 2051)
        self.codebook_eos = raw.get("codebook_eos_token_id", 0)
        self.audio_token_id = raw.get("audio_token_id", 128002)
        self.audio_eos_token_id = raw.get("audio_eos_token_id", 128003)

        def t(n):
            w = get(n)
            if w is None:
                raise KeyError(n)
            return w.to(self.device).to(dtype)

        self.text_embed = t("embed_text_tokens.weight")
        self.audio_embed = t("backbone_model.embed_tokens.embed_audio_tokens.weight")
        self.lm_head = t("lm_head.weight")
        self.backbone = _Decoder(CsmDecoderConfig.from_hf(raw), t, "backbone_model.")
        depth_raw = raw["depth_decoder_config"]
        self.depth = _Decoder(CsmDecoderConfig.from_hf(depth_raw), t, "depth_decoder.model.")
        tied = get("depth_decoder.model.embed_tokens.weight")
        self.depth_embed = self.audio_embed if tied is None else tied.to(self.device).to(dtype)
        self.depth_in = t("depth_decoder.model.inputs_embeds_projector.weight")
        self.depth_heads = t("depth_decoder.codebooks_head.weight")              # [codebooks - 1, hidden, vocab]
        self.codec = Mimi(MimiConfig.from_hf(raw.get("codec_config", {})), get, device, dtype, prefix="codec_model.") \
            if get("codec_model.decoder.layers.0.conv.weight") is not None else None
        self.sampling_rate = raw.get("codec_config", {}).get("sampling_rate", 24000)
        self._offsets = torch.arange(self.codebooks, device=self.device) * self.vocab

    # ------------------------------------------------------------------ inputs
    def frame_embeddings(self, frames: torch.Tensor) -> torch.Tensor:
        """codes [..., codebooks] -> one backbone embedding per frame [..., hidden]."""
        return self.audio_embed[frames.to(self.device).long() + self._offsets].sum(-2)

    @torch.no_grad()
    def prompt_embeddings(self, input_ids: torch.Tensor, context_audio: Optional[list] = None) -> torch.Tensor:
        """input_ids [T] (text ids, ``audio_token_id`` placeholders, ``audio_eos_token_id`` marks) -> [1, T, hidden].
        ``context_audio``: one waveform per run of placeholders, in order; each run must be as long as its frame count."""
        ids = input_ids.to(self.device).long()
        x = self.text_embed[ids].clone()
        slots = (ids == self.audio_token_id).nonzero().flatten()
        if slots.numel():
            if not context_audio or self.codec is None:
                raise ValueError("the prompt has audio positions but no context audio (or no codec) was given")
            frames = torch.cat([self.codec.encode(w.reshape(1, 1, -1))[0].t() for w in context_audio], 0)
            if frames.shape[0] != slots.numel():
                raise ValueError(f"{slots.numel()} audio positions for {frames.shape[0]} audio frames")
            x[slots] = self.frame_embeddings(frames)
        eos = ids == self.audio_eos_token_id
        if eos.any():
            x[eos] = self.frame_embeddings(torch.full((self.codebooks,), self.codebook_eos, device=self.device))
        return x[None]

    # ------------------------------------------------------------------ one frame
    def _pick(self, logits: torch.Tensor, sample: bool, temperature: float, top_k: int, gen) -> torch.Tensor:
        if not sample:
            return logits.argmax(-1)
        logits = logits.float() / max(temperature, 1e-6)
        if 0 < top_k < logits.shape[-1]:
            logits = logits.masked_fill(logits < logits.topk(top_k, -1).values[..., -1:], float("-inf"))
        return torch.multinomial(F.softmax(logits, -1).cpu(), 1, generator=gen)[:, 0].to(logits.device)

    @torch.no_grad()
    def depth_frame(self, hidden: torch.Tensor, first: torch.Tensor, sample=False, temperature=0.9, top_k=50, gen=None) -> torch.Tensor:
        """backbone state [B, H] + codebook-0 tokens [B] -> the whole frame [B, codebooks]."""
        cache = self.depth.new_cache()
        tokens = [first]
        x = torch.stack([hidden, self.depth_embed[first]], 1)                       # positions 0 and 1
        for j in range(1, self.codebooks):
            h = self.depth(F.linear(x, self.depth_in), cache)[:, -1]
            tok = self._pick(h @ self.depth_heads[j - 1], sample, temperature, top_k, gen)
            tokens.append(tok)
            x = self.depth_embed[tok + j * self.vocab][:, None]
        return torch.stack(tokens, 1)

    @torch.no_grad()
    def generate_codes(self, input_ids: torch.Tensor, context_audio: Optional[list] = None, max_frames: int = 125, sample: bool = False,
                       temperature: float = 0.9, top_k: int = 50, seed: int = 0) -> torch.Tensor:
        """-> frames [n, codebooks] (without the closing all-eos frame)."""
        gen = torch.Generator().manual_seed(seed)
        cache = self.backbone.new_cache()
        x = self.prompt_embeddings(input_ids, context_audio)
        frames = []
        for _ in range(max_frames):
            h = self.backbone(x, cache)[:, -1]
            first = self._pick(F.linear(h, self.lm_head), sample, temperature, top_k, gen)
            frame = self.depth_frame(h, first, sample, temperature, top_k, gen)
            if bool((frame == self.codebook_eos).all()):
                break
            frames.append(frame[0])
            x = self.frame_embeddings(frame)[:, None]
        return torch.stack(frames) if frames else torch.zeros(0, self.codebooks, dtype=torch.long, device=self.device)

    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, context_audio: Optional[list] = None, **kw) -> torch.Tensor:
        """-> mono wave [samples] at ``sampling_rate``."""
        if self.codec is None:
            raise ValueError("this checkpoint carries no codec_model.* weights")
        frames = self.generate_codes(input_ids, context_audio, **kw)
        if frames.shape[0] == 0:
            return torch.zeros(0)
        return self.codec.decode(frames.t()[None])[0, 0].float()
