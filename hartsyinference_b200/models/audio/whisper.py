"""Whisper encoder-decoder transformer.

Encoder: two 1-D convolutions over the log-mel frames (kernel 3; the second with stride 2), run as
tap-unfolded GEMMs, fixed sinusoidal positions, bidirectional pre-LayerNorm blocks. Decoder: token +
learned position embeddings, causal self-attention with a growing key/value cache, cross-attention
whose keys and values are projected from the encoder output once per utterance, GELU MLPs, logits
through the tied token embedding.

Reference: src/HartsyInference.Audio/Models/Whisper/, src/HartsyInference.Audio/Pipelines/WhisperPipeline.cs.
Tensor names follow Hugging Face ``WhisperForConditionalGeneration`` (``model.encoder.*``, ``model.decoder.*``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch

from ... import ops
from ..dit.common import WeightFactory


@dataclass(frozen=True)
class WhisperConfig:
    n_mels: int = 80
    width: int = 384
    enc_layers: int = 4
    dec_layers: int = 4
    heads: int = 6
    ffn: int = 1536
    vocab: int = 51865
    max_source: int = 1500
    max_target: int = 448
    eps: float = 1e-5


def tiny_whisper() -> WhisperConfig:
    return WhisperConfig(n_mels=16, width=128, enc_layers=2, dec_layers=2, heads=2, ffn=256, vocab=320,
                         max_source=50, max_target=32)


def whisper_from_hf(d: dict) -> WhisperConfig:
    return WhisperConfig(n_mels=int(d.get("num_mel_bins", 80)), width=int(d["d_model"]),
                         enc_layers=int(d["encoder_layers"]), dec_layers=int(d["decoder_layers"]),
                         heads=int(d["encoder_attention_heads"]), ffn=int(d["encoder_ffn_dim"]),
                         vocab=int(d["vocab_size"]), max_source=int(d.get("max_source_positions", 1500)),
                         max_target=int(d.get("max_target_positions", 448)))


def _pad_k(w: torch.Tensor, mult: int = 64) -> torch.Tensor:
    k = w.shape[1]
    kp = -(-k // mult) * mult
    if kp == k:
        return w.contiguous()
    out = torch.zeros(w.shape[0], kp, dtype=w.dtype, device=w.device)
    out[:, :k] = w
    return out


def _gelu(x: torch.Tensor) -> torch.Tensor:
    return torch.nn.functional.gelu(x.float()).to(torch.bfloat16)


class _Conv1dGemm:
    """Conv1d (kernel 3, padding 1, stride s) over [T, C_in] rows as one GEMM on the unfolded taps;
    K is zero-padded to the tensor-core tile."""

    def __init__(self, w: torch.Tensor, b: torch.Tensor, stride: int, device):
        co, ci, kk = w.shape
        self.stride, self.taps, self.ci = stride, kk, ci
        flat = w.permute(0, 2, 1).reshape(co, kk * ci)          # tap-major: [co, (tap, ci)]
        self.w = ops.LinearWeight(_pad_k(flat.to(torch.bfloat16)).to(device), None, b.to(torch.bfloat16).to(device))
        self.k_pad = self.w.weight.shape[1]

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        t = x.shape[0]
        xp = torch.nn.functional.pad(x, (0, 0, 1, 1))
        cols = torch.cat([xp[i: i + t: 1] for i in range(self.taps)], 1)[:: self.stride]
        cols = torch.nn.functional.pad(cols, (0, self.k_pad - cols.shape[1])).contiguous()
        return ops.linear(cols, self.w)


class WhisperModel:
    def __init__(self, cfg: WhisperConfig, device="cpu", get: Optional[Callable[[str], Optional[torch.Tensor]]] = None,
                 seed: int = 0):
        self.cfg, self.device = cfg, torch.device(device)
        W = cfg.width

        def get0(name: str):
            # k_proj has no bias in the checkpoint; the fused qkv wants one of the same length
            t = get(name)
            if t is None and name.endswith("k_proj.bias"):
                return torch.zeros(W)
            return t

        f = WeightFactory(self.device, False, get=get0 if get is not None else None, seed=seed)
        e = "model.encoder."
        self.conv1 = _Conv1dGemm(f.tensor(e + "conv1.weight", W, cfg.n_mels, 3).cpu(), f.tensor(e + "conv1.bias", W).cpu(), 1, self.device)
        self.conv2 = _Conv1dGemm(f.tensor(e + "conv2.weight", W, W, 3).cpu(), f.tensor(e + "conv2.bias", W).cpu(), 2, self.device)
        self.enc_pos = f.tensor(e + "embed_positions.weight", cfg.max_source, W)

        def attn(p: str, cross: bool):
            if cross:
                return dict(q=f.linear(p + "q_proj", W, W), kv=f.linear([p + "k_proj", p + "v_proj"], [W, W], W),
                            o=f.linear(p + "out_proj", W, W))
            return dict(qkv=f.linear([p + "q_proj", p + "k_proj", p + "v_proj"], [W, W, W], W), o=f.linear(p + "out_proj", W, W))

        def ln(p: str):
            return f.tensor(p + ".weight", W, ones=True), f.tensor(p + ".bias", W, zeros=True)

        self.enc = []
        for i in range(cfg.enc_layers):
            p = f"{e}layers.{i}."
            self.enc.append(dict(ln1=ln(p + "self_attn_layer_norm"), attn=attn(p + "self_attn.", False),
                                 ln2=ln(p + "final_layer_norm"), fc1=f.linear(p + "fc1", cfg.ffn, W), fc2=f.linear(p + "fc2", W, cfg.ffn)))
        self.enc_ln = ln(e + "layer_norm")
        d = "model.decoder."
        self.tok = f.tensor(d + "embed_tokens.weight", cfg.vocab, W)
        self.head = ops.LinearWeight(self.tok)
        self.dec_pos = f.tensor(d + "embed_positions.weight", cfg.max_target, W)
        self.dec = []
        for i in range(cfg.dec_layers):
            p = f"{d}layers.{i}."
            self.dec.append(dict(ln1=ln(p + "self_attn_layer_norm"), attn=attn(p + "self_attn.", False),
                                 lnx=ln(p + "encoder_attn_layer_norm"), cross=attn(p + "encoder_attn.", True),
                                 ln2=ln(p + "final_layer_norm"), fc1=f.linear(p + "fc1", cfg.ffn, W), fc2=f.linear(p + "fc2", W, cfg.ffn)))
        self.dec_ln = ln(d + "layer_norm")

    def _ln(self, x, wb):
        return ops.norm(x, wb[0], bias=wb[1], layernorm=True, eps=self.cfg.eps)[0]

    # ------------------------------------------------------------------------------- encoder
    @torch.no_grad()
    def encode(self, mel: torch.Tensor) -> torch.Tensor:
        """mel [n_mels, frames] -> encoder states [frames / 2, W]."""
        cfg = self.cfg
        h, d = cfg.heads, cfg.width // cfg.heads
        x = mel.to(self.device).to(torch.bfloat16).t().contiguous()
        x = _gelu(self.conv1(x))
        x = _gelu(self.conv2(x))
        L = x.shape[0]
        x = (x.float() + self.enc_pos[:L].float()).to(torch.bfloat16)
        for b in self.enc:
            y = self._ln(x, b["ln1"])
            q, k, v = ops.dit_qkv(ops.linear(y, b["attn"]["qkv"]), h, h, d)
            a = ops.attention(q, k, v, causal=False)
            x = ops.linear(a.reshape(L, -1), b["attn"]["o"], residual=x)
            y = self._ln(x, b["ln2"])
            x = ops.linear(_gelu(ops.linear(y, b["fc1"])), b["fc2"], residual=x)
        return self._ln(x, self.enc_ln)

    # ------------------------------------------------------------------------------- decoder
    @torch.no_grad()
    def start(self, enc: torch.Tensor) -> dict:
        """Decoder state for one utterance: cross-attention K/V of every layer and empty self caches."""
        cfg = self.cfg
        h, d = cfg.heads, cfg.width // cfg.heads
        cross = []
        for b in self.dec:
            kv = ops.linear(enc, b["cross"]["kv"]).reshape(enc.shape[0], 2, h, d)
            cross.append((kv[:, 0].contiguous(), kv[:, 1].contiguous()))
        cap = cfg.max_target
        kv = [(torch.zeros(cap, h, d, dtype=torch.bfloat16, device=self.device),
               torch.zeros(cap, h, d, dtype=torch.bfloat16, device=self.device)) for _ in self.dec]
        return dict(cross=cross, kv=kv, pos=0)

    @torch.no_grad()
    def decode(self, state: dict, tokens: torch.Tensor) -> torch.Tensor:
        """Feed ``tokens`` [n] at positions state['pos'].., append to the caches, return logits [n, vocab]."""
        cfg = self.cfg
        h, d = cfg.heads, cfg.width // cfg.heads
        n, p0 = tokens.numel(), state["pos"]
        if p0 + n > cfg.max_target:
            raise ValueError("decoder context exhausted")
        tokens = tokens.to(self.device)
        x = (self.tok[tokens.long()].float() + self.dec_pos[p0:p0 + n].float()).to(torch.bfloat16)
        for b, (ck, cv), (sk, sv) in zip(self.dec, state["cross"], state["kv"]):
            y = self._ln(x, b["ln1"])
            q, k, v = ops.dit_qkv(ops.linear(y, b["attn"]["qkv"]), h, h, d)
            sk[p0:p0 + n], sv[p0:p0 + n] = k, v
            if n == 1:
                a = ops.attention(q, sk[:p0 + 1], sv[:p0 + 1], causal=False)
            elif p0 == 0:
                a = ops.attention(q, k, v, causal=True)
            else:   # a multi-token continuation: one query row at a time keeps the causal mask exact
                a = torch.cat([ops.attention(q[i:i + 1], sk[:p0 + i + 1], sv[:p0 + i + 1], causal=False) for i in range(n)], 0)
            x = ops.linear(a.reshape(n, -1), b["attn"]["o"], residual=x)
            y = self._ln(x, b["lnx"])
            q = ops.linear(y, b["cross"]["q"]).reshape(n, h, d)
            a = ops.attention(q, ck, cv, causal=False)
            x = ops.linear(a.reshape(n, -1), b["cross"]["o"], residual=x)
            y = self._ln(x, b["ln2"])
            x = ops.linear(_gelu(ops.linear(y, b["fc1"])), b["fc2"], residual=x)
        state["pos"] = p0 + n
        return ops.linear(self._ln(x, self.dec_ln), self.head).float()
