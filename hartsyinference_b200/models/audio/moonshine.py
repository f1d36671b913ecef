"""Moonshine speech recognition: an encoder-decoder transformer that reads raw 16 kHz audio.

Front end: three strided 1-D convolutions over the waveform (kernel 127 stride 64 with tanh and a
GroupNorm, then kernel 7 stride 3 and kernel 3 stride 2 with GELU: one frame per 384 samples).
Encoder blocks: pre-LayerNorm (no bias), self-attention with interleaved rotary embedding on the
first 90 % of each head, GELU MLP. Decoder blocks: causal self-attention with the same rotary
scheme and a key / value cache, cross-attention over the encoder states (projected once per
utterance), SiLU-gated MLP. Logits through the tied token embedding.

The models are small (27 M / 61 M parameters) with head sizes outside the tensor-core attention
kernels' set, so this runs on plain PyTorch ops on whichever device holds the weights.

Reference: src/HartsyInference.Audio/Models/Moonshine/, Pipelines/MoonshinePipeline.cs.
Tensor names follow Hugging Face ``MoonshineForConditionalGeneration``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.nn.functional as F


@dataclass(frozen=True)
class MoonshineConfig:
    vocab_size: int = 32768
    hidden: int = 288
    ffn: int = 1152
    enc_layers: int = 6
    dec_layers: int = 6
    heads: int = 8
    rotary_factor: float = 0.9
    theta: float = 10000.0
    bos_id: int = 1
    eos_id: int = 2
    max_positions: int = 512

    @property
    def head_dim(self) -> int:
        return self.hidden // self.heads

    @property
    def rot(self) -> int:
        return int(self.head_dim * self.rotary_factor) // 2 * 2


def tiny_moonshine() -> MoonshineConfig:
    return MoonshineConfig(vocab_size=300, hidden=64, ffn=128, enc_layers=2, dec_layers=2, heads=2, max_positions=128)


def moonshine_from_hf(d: dict) -> MoonshineConfig:
    rp = d.get("rope_parameters") or {}
    return MoonshineConfig(vocab_size=d["vocab_size"], hidden=d["hidden_size"], ffn=d["intermediate_size"],
                           enc_layers=d["encoder_num_hidden_layers"], dec_layers=d["decoder_num_hidden_layers"],
                           heads=d["encoder_num_attention_heads"],
                           rotary_factor=float(d.get("partial_rotary_factor") or rp.get("partial_rotary_factor") or 0.9),
                           theta=float(d.get("rope_theta") or rp.get("rope_theta") or 10000.0), bos_id=d.get("decoder_start_token_id", 1),
                           eos_id=d.get("eos_token_id", 2), max_positions=d.get("max_position_embeddings", 512))


class MoonshineModel:
    def __init__(self, cfg: MoonshineConfig, device="cpu", get: Optional[Callable[[str], Optional[torch.Tensor]]] = None, seed: int = 0):
        self.cfg, self.device = cfg, torch.device(device)
        self._get = get
        self._g = torch.Generator().manual_seed(seed)
        self.w: dict[str, torch.Tensor] = {}
        self.inv_freq = (cfg.theta ** (-torch.arange(0, cfg.rot, 2, dtype=torch.float32) / cfg.rot)).to(self.device)

    def p(self, name: str, *shape, ones: bool = False, zeros: bool = False) -> torch.Tensor:
        t = self.w.get(name)
        if t is None:
            t = self._get(name) if self._get is not None else None
            if t is None:
                if self._get is not None:
                    raise KeyError(name)
                fan = 1
                for s in shape[1:]:
                    fan *= s
                t = torch.ones(*shape) if ones else torch.zeros(*shape) if zeros else torch.randn(*shape, generator=self._g) * (1.0 / max(fan, 1)) ** 0.5
            t = t.float().to(self.device)
            self.w[name] = t
        return t

    def _ln(self, x, name):
        H = self.cfg.hidden
        return F.layer_norm(x, (H,), self.p(name + ".weight", H, ones=True), None, 1e-5)

    def _lin(self, x, name, o, i, bias=False):
        return F.linear(x, self.p(name + ".weight", o, i), self.p(name + ".bias", o, zeros=True) if bias else None)

    def _rope(self, x: torch.Tensor, pos0: int) -> torch.Tensor:
        """x [T, heads, d]: rotate interleaved pairs of the first ``rot`` channels."""
        rot = self.cfg.rot
        T = x.shape[0]
        ang = (torch.arange(pos0, pos0 + T, device=x.device, dtype=torch.float32)[:, None] * self.inv_freq[None])[:, None, :]
        cos, sin = ang.cos(), ang.sin()
        a, b = x[..., 0:rot:2], x[..., 1:rot:2]
        out = torch.stack([a * cos - b * sin, b * cos + a * sin], -1).flatten(-2)
        return torch.cat([out, x[..., rot:]], -1)

    def _attend(self, q, k, v, causal_from: Optional[int] = None):
        """q [Tq, h, d], k / v [Tk, h, d] -> [Tq, h * d]; ``causal_from`` = position of the first query."""
        qh, kh, vh = q.transpose(0, 1), k.transpose(0, 1), v.transpose(0, 1)
        mask = None
        if causal_from is not None and q.shape[0] > 1:
            qi = torch.arange(causal_from, causal_from + q.shape[0], device=q.device)[:, None]
            mask = torch.arange(k.shape[0], device=q.device)[None, :] <= qi
        o = F.scaled_dot_product_attention(qh[None], kh[None], vh[None], attn_mask=mask)[0]
        return o.transpose(0, 1).reshape(q.shape[0], -1)

    # ------------------------------------------------------------------------------- encoder
    @torch.no_grad()
    def encode(self, audio: torch.Tensor) -> torch.Tensor:
        """audio [n] float at 16 kHz -> encoder states [frames, H]."""
        cfg = self.cfg
        H, h, d = cfg.hidden, cfg.heads, cfg.head_dim
        x = audio.to(self.device).float()[None, None]
        x = torch.tanh(F.conv1d(x, self.p("model.encoder.conv1.weight", H, 1, 127), None, stride=64))
        x = F.group_norm(x, 1, self.p("model.encoder.groupnorm.weight", H, ones=True), self.p("model.encoder.groupnorm.bias", H, zeros=True), 1e-5)
        x = F.gelu(F.conv1d(x, self.p("model.encoder.conv2.weight", 2 * H, H, 7), self.p("model.encoder.conv2.bias", 2 * H, zeros=True), stride=3))
        x = F.gelu(F.conv1d(x, self.p("model.encoder.conv3.weight", H, 2 * H, 3), self.p("model.encoder.conv3.bias", H, zeros=True), stride=2))
        x = x[0].t()
        T = x.shape[0]
        for i in range(cfg.enc_layers):
            p = f"model.encoder.layers.{i}."
            y = self._ln(x, p + "input_layernorm")
            q = self._rope(self._lin(y, p + "self_attn.q_proj", H, H).reshape(T, h, d), 0)
            k = self._rope(self._lin(y, p + "self_attn.k_proj", H, H).reshape(T, h, d), 0)
            v = self._lin(y, p + "self_attn.v_proj", H, H).reshape(T, h, d)
            x = x + self._lin(self._attend(q, k, v), p + "self_attn.o_proj", H, H)
            y = self._ln(x, p + "post_attention_layernorm")
            x = x + self._lin(F.gelu(self._lin(y, p + "mlp.fc1", cfg.ffn, H, True)), p + "mlp.fc2", H, cfg.ffn, True)
        return self._ln(x, "model.encoder.layer_norm")

    # ------------------------------------------------------------------------------- decoder
    @torch.no_grad()
    def start(self, enc: torch.Tensor) -> dict:
        cfg = self.cfg
        H, h, d = cfg.hidden, cfg.heads, cfg.head_dim
        cross = []
        for i in range(cfg.dec_layers):
            p = f"model.decoder.layers.{i}.encoder_attn."
            cross.append((self._lin(enc, p + "k_proj", H, H).reshape(-1, h, d), self._lin(enc, p + "v_proj", H, H).reshape(-1, h, d)))
        return dict(cross=cross, k=[None] * cfg.dec_layers, v=[None] * cfg.dec_layers, pos=0)

    @torch.no_grad()
    def decode(self, st: dict, tokens: torch.Tensor) -> torch.Tensor:
        """tokens [n] at positions st['pos'].. -> logits [n, vocab]; the caches grow by n."""
        cfg = self.cfg
        H, h, d = cfg.hidden, cfg.heads, cfg.head_dim
        n, p0 = tokens.numel(), st["pos"]
        emb = self.p("model.decoder.embed_tokens.weight", cfg.vocab_size, H)
        x = emb[tokens.long().to(self.device)]
        for i in range(cfg.dec_layers):
            p = f"model.decoder.layers.{i}."
            y = self._ln(x, p + "input_layernorm")
            q = self._rope(self._lin(y, p + "self_attn.q_proj", H, H).reshape(n, h, d), p0)
            k = self._rope(self._lin(y, p + "self_attn.k_proj", H, H).reshape(n, h, d), p0)
            v = self._lin(y, p + "self_attn.v_proj", H, H).reshape(n, h, d)
            st["k"][i] = k if st["k"][i] is None else torch.cat([st["k"][i], k], 0)
            st["v"][i] = v if st["v"][i] is None else torch.cat([st["v"][i], v], 0)
            x = x + self._lin(self._attend(q, st["k"][i], st["v"][i], causal_from=p0), p + "self_attn.o_proj", H, H)
            y = self._ln(x, p + "post_attention_layernorm")
            q = self._lin(y, p + "encoder_attn.q_proj", H, H).reshape(n, h, d)
            ck, cv = st["cross"][i]
            x = x + self._lin(self._attend(q, ck, cv), p + "encoder_attn.o_proj", H, H)
            y = self._ln(x, p + "final_layernorm")
            up, gate = self._lin(y, p + "mlp.fc1", 2 * cfg.ffn, H, True).chunk(2, -1)
            x = x + self._lin(F.silu(gate) * up, p + "mlp.fc2", H, cfg.ffn, True)
        st["pos"] = p0 + n
        return F.linear(self._ln(x, "model.decoder.norm"), emb)

    @torch.no_grad()
    def transcribe_tokens(self, audio: torch.Tensor, max_tokens: Optional[int] = None) -> list[int]:
        """Greedy decoding; the token budget follows the audio length (about 6.5 tokens per second)."""
        cfg = self.cfg
        limit = max_tokens or max(1, int(audio.numel() / 16000 * 6.5) + 1)
        limit = min(limit, cfg.max_positions - 1)
        st = self.start(self.encode(audio))
        tok, out = cfg.bos_id, []
        for _ in range(limit):
            tok = int(self.decode(st, torch.tensor([tok]))[-1].argmax())
            if tok == cfg.eos_id:
                break
            out.append(tok)
        return out
