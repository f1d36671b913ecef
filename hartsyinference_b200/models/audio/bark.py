"""Bark: text -> speech through three token language models and the EnCodec decoder.

1. *semantic* (causal GPT, learned positions): the input is 256 text positions, each the sum of the
   text-token embedding (ids offset into the upper part of the table, padded) and the embedding of a
   semantic-history token (padding when there is no voice prompt), followed by one "infer" token.
   It samples semantic tokens (50 Hz worth of content at 49.9 tokens / s) until the end token wins:
   only ids below the semantic vocabulary and the end token may be drawn, and once the end token's
   probability passes ``min_eos_p`` it is forced.
2. *coarse* (same architecture): from a window of semantic tokens (right-padded to 256) + an infer
   token + the coarse tokens so far, it emits the first two EnCodec codebooks interleaved frame by
   frame (75 Hz x 2); step parity picks which codebook's id range is allowed. Long utterances
   advance in sliding windows of 60 tokens over at most 630 tokens of coarse history.
3. *fine* (the same blocks without the causal mask, one embedding table and one output head per
   codebook): codebook k of a 1024-frame window is predicted from the sum of the embeddings of
   codebooks 0..k, for k = 2..7, windows advancing by 512 frames.

The 8 x frames code matrix goes through the EnCodec quantiser tables and decoder (24 kHz).
Weights use the names of the converted checkpoints (``semantic.*``, ``coarse_acoustics.*``,
``fine_acoustics.*``, ``codec_model.*``). Reference: src/HartsyInference.Audio/Models/Bark/,
Pipelines/BarkPipeline.cs.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, Optional

import torch
import torch.nn.functional as F

from .encodec import EncodecConfig, EncodecDecoder


@dataclass(frozen=True)
class BarkGptConfig:
    hidden: int = 1024
    layers: int = 24
    heads: int = 16
    block_size: int = 1024
    input_vocab: int = 10048
    output_vocab: int = 10048
    bias: bool = False
    codes_total: int = 8             # fine model only
    codes_given: int = 1

    @staticmethod
    def from_hf(d: dict) -> "BarkGptConfig":
        return BarkGptConfig(hidden=d.get("hidden_size", 1024), layers=d.get("num_layers", 24), heads=d.get("num_heads", 16),
                             block_size=d.get("block_size", 1024), input_vocab=d.get("input_vocab_size", 10048),
                             output_vocab=d.get("output_vocab_size", 10048), bias=bool(d.get("bias", False)),
                             codes_total=d.get("n_codes_total", 8), codes_given=d.get("n_codes_given", 1))


@dataclass
class BarkGenerationConfig:
    """The token bookkeeping of the three stages (defaults of the released checkpoints)."""
    text_encoding_offset: int = 10048
    text_pad_token: int = 129595
    semantic_vocab_size: int = 10000
    semantic_pad_token: int = 10000          # also the end token of the semantic stage
    semantic_infer_token: int = 129599
    max_input_semantic_length: int = 256
    semantic_rate_hz: float = 49.9
    semantic_max_new_tokens: int = 768
    min_eos_p: Optional[float] = None
    semantic_temperature: float = 1.0
    coarse_semantic_pad_token: int = 12048
    coarse_infer_token: int = 12050
    coarse_rate_hz: int = 75
    n_coarse_codebooks: int = 2
    n_fine_codebooks: int = 8
    max_coarse_input_length: int = 256
    max_coarse_history: int = 630
    sliding_window_len: int = 60
    coarse_temperature: float = 1.0
    max_fine_history_length: int = 512
    max_fine_input_length: int = 1024
    fine_temperature: float = 1.0
    codebook_size: int = 1024

    @staticmethod
    def from_hf(d: dict) -> "BarkGenerationConfig":
        g = BarkGenerationConfig()
        s, c, f = d.get("semantic_config", {}), d.get("coarse_acoustics_config", {}), d.get("fine_acoustics_config", {})
        for src, pairs in ((s, (("text_encoding_offset",) * 2, ("text_pad_token",) * 2, ("semantic_vocab_size",) * 2,
                                ("semantic_pad_token",) * 2, ("semantic_infer_token",) * 2, ("max_input_semantic_length",) * 2,
                                ("semantic_rate_hz",) * 2, ("max_new_tokens", "semantic_max_new_tokens"), ("min_eos_p",) * 2,
                                ("temperature", "semantic_temperature"))),
                           (c, (("coarse_semantic_pad_token",) * 2, ("coarse_infer_token",) * 2, ("coarse_rate_hz",) * 2,
                                ("n_coarse_codebooks",) * 2, ("max_coarse_input_length",) * 2, ("max_coarse_history",) * 2,
                                ("sliding_window_len",) * 2, ("temperature", "coarse_temperature"))),
                           (f, (("n_fine_codebooks",) * 2, ("max_fine_history_length",) * 2, ("max_fine_input_length",) * 2,
                                ("temperature", "fine_temperature")))):
            for key, attr in pairs:
                if src.get(key) is not None:
                    setattr(g, attr, src[key])
        g.codebook_size = d.get("codebook_size", 1024)
        return g

    @property
    def semantic_to_coarse(self) -> float:
        return self.coarse_rate_hz / self.semantic_rate_hz * self.n_coarse_codebooks


class BarkGpt:
    """One of the three transformers. ``causal`` False builds the fine model (per-codebook tables and heads)."""

    def __init__(self, cfg: BarkGptConfig, get: Callable[[str], Optional[torch.Tensor]], prefix: str, device="cpu",
                 dtype: torch.dtype = torch.float32, causal: bool = True):
        self.cfg, self.device, self.dtype, self.causal = cfg, torch.device(device), dtype, causal

        def t(n, optional=False):
            w = get(prefix + n)
            if w is None:
                if optional:
                    return None
                raise KeyError(prefix + n)
            return w.to(self.device).to(dtype)

        self.pos = t("position_embeds_layer.weight")
        if causal:
            self.embed = [t("input_embeds_layer.weight")]
            self.heads_w = [t("lm_head.weight")]
        else:
            self.embed = [t(f"input_embeds_layers.{i}.weight") for i in range(cfg.codes_total)]
            # a head is stored, or shares the table of the codebook it predicts
            self.heads_w = []
            for i in range(cfg.codes_total - cfg.codes_given):
                w = t(f"lm_heads.{i}.weight", optional=True)
                self.heads_w.append(w if w is not None else self.embed[i + 1])
        self.blocks = []
        for i in range(cfg.layers):
            p = f"layers.{i}."
            self.blocks.append({
                "ln1": (t(p + "layernorm_1.weight"), t(p + "layernorm_1.bias", True)),
                "ln2": (t(p + "layernorm_2.weight"), t(p + "layernorm_2.bias", True)),
                "qkv": (t(p + "attn.att_proj.weight"), t(p + "attn.att_proj.bias", True)),
                "out": (t(p + "attn.out_proj.weight"), t(p + "attn.out_proj.bias", True)),
                "up": (t(p + "mlp.in_proj.weight"), t(p + "mlp.in_proj.bias", True)),
                "down": (t(p + "mlp.out_proj.weight"), t(p + "mlp.out_proj.bias", True)),
            })
        self.ln_f = (t("layernorm_final.weight"), t("layernorm_final.bias", True))

    def new_cache(self) -> dict:
        return {"k": [None] * self.cfg.layers, "v": [None] * self.cfg.layers, "len": 0}

    def hidden(self, x: torch.Tensor, cache: Optional[dict] = None) -> torch.Tensor:
        """x [B, T, H] token embeddings (positions are added here) -> final-norm states [B, T, H]."""
        cfg = self.cfg
        b, t, h = x.shape
        past = cache["len"] if cache is not None else 0
        x = x + self.pos[past:past + t]
        hd = h // cfg.heads
        for i, blk in enumerate(self.blocks):
            y = F.layer_norm(x, (h,), *blk["ln1"])
            q, k, v = F.linear(y, *blk["qkv"]).view(b, t, 3, cfg.heads, hd).permute(2, 0, 3, 1, 4)
            if cache is not None:
                if cache["k"][i] is not None:
                    k, v = torch.cat([cache["k"][i], k], 2), torch.cat([cache["v"][i], v], 2)
                cache["k"][i], cache["v"][i] = k, v
            a = F.scaled_dot_product_attention(q, k, v, is_causal=self.causal and t > 1)
            x = x + F.linear(a.transpose(1, 2).reshape(b, t, h), *blk["out"])
            y = F.layer_norm(x, (h,), *blk["ln2"])
            x = x + F.linear(F.gelu(F.linear(y, *blk["up"])), *blk["down"])
        if cache is not None:
            cache["len"] = past + t
        return F.layer_norm(x, (h,), *self.ln_f)

    def logits(self, ids: Optional[torch.Tensor] = None, embeds: Optional[torch.Tensor] = None, cache: Optional[dict] = None,
               last_only: bool = False) -> torch.Tensor:
        """Causal stages: ids [B, T] (or ready embeddings) -> logits [B, T, vocab] in fp32."""
        x = self.embed[0][ids.to(self.device)] if embeds is None else embeds
        hs = self.hidden(x, cache)
        if last_only:
            hs = hs[:, -1:]
        return F.linear(hs, self.heads_w[0]).float()

    def fine_logits(self, codebook: int, codes: torch.Tensor) -> torch.Tensor:
        """codes [B, T, codes_total] -> logits [B, T, vocab] for ``codebook`` from the tables of codebooks 0..codebook."""
        codes = codes.to(self.device).long()
        x = sum(self.embed[i][codes[:, :, i]] for i in range(codebook + 1))
        return F.linear(self.hidden(x), self.heads_w[codebook - self.cfg.codes_given]).float()


def _draw(logits: torch.Tensor, temperature: float, sample: bool, gen: Optional[torch.Generator]) -> torch.Tensor:
    if not sample:
        return logits.argmax(-1)
    p = F.softmax(logits / max(temperature, 1e-6), -1)
    return torch.multinomial(p.cpu(), 1, generator=gen)[:, 0].to(logits.device)


class Bark:
    def __init__(self, raw: dict, get: Callable[[str], Optional[torch.Tensor]], device="cpu", dtype: torch.dtype = torch.float32,
                 generation: Optional[dict] = None):
        self.device = torch.device(device)
        self.gen = BarkGenerationConfig.from_hf(generation or {})
        self.semantic = BarkGpt(BarkGptConfig.from_hf(raw.get("semantic_config", {})), get, "semantic.", device, dtype)
        self.coarse = BarkGpt(BarkGptConfig.from_hf(raw.get("coarse_acoustics_config", {})), get, "coarse_acoustics.", device, dtype)
        self.fine = BarkGpt(BarkGptConfig.from_hf(raw.get("fine_acoustics_config", {})), get, "fine_acoustics.", device, dtype,
                            causal=False)
        codec_raw = raw.get("codec_config", {})
        sub = lambda n: get("codec_model." + n)
        self.codec = EncodecDecoder(EncodecConfig.from_hf(codec_raw), sub, device) if sub("decoder.layers.0.conv.weight_g") is not None \
            or sub("decoder.layers.0.conv.parametrizations.weight.original0") is not None else None
        self.sampling_rate = codec_raw.get("sampling_rate", 24000)

    # ------------------------------------------------------------------ stage 1
    @torch.no_grad()
    def semantic_tokens(self, text_ids: torch.Tensor, history: Optional[dict] = None, sample: bool = True,
                        seed: int = 0, max_new_tokens: Optional[int] = None) -> torch.Tensor:
        """text_ids [T] (tokenizer ids, before the offset) -> semantic tokens [n] (without the end token)."""
        g, m = self.gen, self.semantic
        n_in = g.max_input_semantic_length
        ids = text_ids.to(self.device).long()[:n_in] + g.text_encoding_offset
        ids = F.pad(ids, (0, n_in - ids.numel()), value=g.text_pad_token)
        if history is not None:
            hist = history["semantic_prompt"].to(self.device).long()[-n_in:]
            hist = F.pad(hist, (0, n_in - hist.numel()), value=g.semantic_pad_token)
        else:
            hist = torch.full((n_in,), g.semantic_pad_token, device=self.device, dtype=torch.long)
        infer = torch.tensor([g.semantic_infer_token], device=self.device)
        x = torch.cat([m.embed[0][ids] + m.embed[0][hist], m.embed[0][infer]], 0)[None]
        rng = torch.Generator().manual_seed(seed)
        cache = m.new_cache()
        logits = m.logits(embeds=x, cache=cache, last_only=True)[:, -1]
        out = []
        limit = max_new_tokens or g.semantic_max_new_tokens
        for _ in range(limit):
            logits[:, g.semantic_vocab_size:g.semantic_pad_token] = -math.inf
            logits[:, g.semantic_pad_token + 1:] = -math.inf
            if g.min_eos_p and float(F.softmax(logits, -1)[0, g.semantic_pad_token]) > g.min_eos_p:
                break
            tok = _draw(logits, g.semantic_temperature, sample, rng)
            if int(tok) == g.semantic_pad_token:
                break
            out.append(int(tok))
            if cache["len"] + 1 > m.cfg.block_size:
                break
            logits = m.logits(ids=tok[None], cache=cache, last_only=True)[:, -1]
        return torch.tensor(out, dtype=torch.long, device=self.device)

    # ------------------------------------------------------------------ stage 2
    def _histories(self, history: Optional[dict]):
        g = self.gen
        if history is None:
            e = torch.zeros(0, dtype=torch.long, device=self.device)
            return e, e
        sem = history["semantic_prompt"].to(self.device).long()
        co = history["coarse_prompt"].to(self.device).long().clone()
        co += (torch.arange(co.shape[0], device=self.device) * g.codebook_size)[:, None]
        co = co.t().reshape(-1) + g.semantic_vocab_size
        ratio = g.semantic_to_coarse
        max_sem = int(math.floor(g.max_coarse_history / ratio))
        n_sem = min(max_sem, sem.numel() - sem.numel() % 2, int(math.floor(co.numel() / ratio)))
        n_co = int(round(n_sem * ratio))
        sem = sem[sem.numel() - n_sem:] if n_sem else sem[:0]
        co = co[co.numel() - n_co:] if n_co else co[:0]
        return sem, co[:-2]                  # two tokens dropped for time alignment, as the model was used in training

    @torch.no_grad()
    def coarse_tokens(self, semantic: torch.Tensor, history: Optional[dict] = None, sample: bool = True, seed: int = 0) -> torch.Tensor:
        """semantic [n] -> coarse tokens [2 * frames] (first / second codebook interleaved, in the coarse model's id space)."""
        g, m = self.gen, self.coarse
        ratio = g.semantic_to_coarse
        max_sem_hist = int(math.floor(g.max_coarse_history / ratio))
        semantic = semantic.to(self.device).long().clone()
        semantic[semantic == g.semantic_pad_token] = g.coarse_semantic_pad_token
        n_real = int((semantic != g.coarse_semantic_pad_token).sum())
        total = int(round(math.floor(n_real * ratio / g.n_coarse_codebooks) * g.n_coarse_codebooks))
        sem_hist, x_coarse = self._histories(history)
        base = sem_hist.numel()
        semantic = torch.cat([sem_hist, semantic])
        n_hist = x_coarse.numel()
        rng = torch.Generator().manual_seed(seed + 1)
        done = 0
        while done < total:
            idx = base + int(round(done / ratio))
            window = semantic[max(0, idx - max_sem_hist):][:g.max_coarse_input_length]
            window = F.pad(window, (0, g.max_coarse_input_length - window.numel()), value=g.coarse_semantic_pad_token)
            prompt = torch.cat([window, torch.tensor([g.coarse_infer_token], device=self.device), x_coarse[-g.max_coarse_history:]])
            cache = m.new_cache()
            logits = m.logits(ids=prompt[None], cache=cache, last_only=True)[:, -1]
            steps = min(g.sliding_window_len, total - done)
            new = []
            for s in range(steps):
                first = s % 2 == 0                      # windows hold whole frames, so parity restarts with each
                lo = g.semantic_vocab_size + (0 if first else g.codebook_size)
                masked = torch.full_like(logits, -math.inf)
                hi = lo + g.codebook_size if first else logits.shape[-1]
                masked[:, lo:hi] = logits[:, lo:hi]
                tok = _draw(masked, g.coarse_temperature, sample, rng)
                new.append(int(tok))
                if s + 1 < steps:
                    logits = m.logits(ids=tok[None], cache=cache, last_only=True)[:, -1]
            x_coarse = torch.cat([x_coarse, torch.tensor(new, dtype=torch.long, device=self.device)])
            done = x_coarse.numel() - n_hist
        return x_coarse[n_hist:]

    # ------------------------------------------------------------------ stage 3
    @torch.no_grad()
    def fine_codes(self, coarse: torch.Tensor, history: Optional[dict] = None, sample: bool = False, seed: int = 0) -> torch.Tensor:
        """coarse [2 * frames] -> codes [n_fine_codebooks, frames] (ids in [0, codebook_size))."""
        g, m = self.gen, self.fine
        n_co, n_fine, size = g.n_coarse_codebooks, g.n_fine_codebooks, g.codebook_size
        co = torch.remainder(coarse.to(self.device).long().view(-1, n_co) - g.semantic_vocab_size, size)
        frames = co.shape[0]
        buf = F.pad(co, (0, n_fine - n_co), value=size)
        n_history = 0
        if history is not None:
            h = history["fine_prompt"].to(self.device).long().t()[-g.max_fine_history_length:]
            buf, n_history = torch.cat([h, buf], 0), h.shape[0]
        trim = 0
        if buf.shape[0] < g.max_fine_input_length:
            trim = g.max_fine_input_length - buf.shape[0]
            buf = F.pad(buf, (0, 0, 0, trim), value=size)
        loops = max(0, int(math.ceil((frames - (g.max_fine_input_length - n_history)) / g.max_fine_history_length))) + 1
        rng = torch.Generator().manual_seed(seed + 2)
        for n in range(loops):
            start = min(n * g.max_fine_history_length, buf.shape[0] - g.max_fine_input_length)
            fill = min(n_history + n * g.max_fine_history_length, buf.shape[0] - g.max_fine_history_length)
            rel = fill - start
            window = buf[start:start + g.max_fine_input_length].clone()
            for k in range(n_co, n_fine):
                logits = m.fine_logits(k, window[None])[0, rel:, :size]
                if sample and g.fine_temperature != 1.0:
                    pred = torch.multinomial(F.softmax(logits / g.fine_temperature, -1).cpu(), 1, generator=rng)[:, 0].to(self.device)
                else:
                    pred = logits.argmax(-1)
                window[rel:, k] = pred
            buf[fill:fill + (g.max_fine_input_length - rel), n_co:] = window[rel:, n_co:]
        out = buf.t()[:, n_history:]
        if trim:
            out = out[:, :-trim]
        assert out.shape[1] == frames
        return out

    # ------------------------------------------------------------------ all of it
    @torch.no_grad()
    def generate_codes(self, text_ids: torch.Tensor, history: Optional[dict] = None, sample: bool = True, seed: int = 0,
                       max_semantic_tokens: Optional[int] = None) -> torch.Tensor:
        sem = self.semantic_tokens(text_ids, history, sample, seed, max_semantic_tokens)
        if sem.numel() == 0:
            return torch.zeros(self.gen.n_fine_codebooks, 0, dtype=torch.long, device=self.device)
        return self.fine_codes(self.coarse_tokens(sem, history, sample, seed), history, sample, seed)

    @torch.no_grad()
    def generate(self, text_ids: torch.Tensor, history: Optional[dict] = None, sample: bool = True, seed: int = 0,
                 max_semantic_tokens: Optional[int] = None) -> torch.Tensor:
        """-> mono wave [samples] at ``sampling_rate``."""
        if self.codec is None:
            raise ValueError("this checkpoint carries no codec_model.* weights")
        codes = self.generate_codes(text_ids, history, sample, seed, max_semantic_tokens)
        if codes.shape[1] == 0:
            return torch.zeros(0)
        return self.codec.decode(codes[None])[0, 0].float()
