"""BERT-family sentence-embedding encoder (post-LayerNorm blocks, learned position and token-type
embeddings, exact GELU), pooled by CLS token or attention-masked mean and L2-normalised.

Reference: src/HartsyInference.LLM/Embeddings/BertEmbeddingModel.cs and
src/HartsyInference.ModelAssets/TextEncoders/Bert (weight mapping; Hugging Face ``BertModel`` names
with or without the ``bert.`` prefix).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch

from ... import ops
from ..dit.common import WeightFactory


@dataclass(frozen=True)
class BertConfig:
    vocab_size: int = 30522
    hidden: int = 768
    layers: int = 12
    heads: int = 12
    intermediate: int = 3072
    max_len: int = 512
    type_vocab: int = 2
    eps: float = 1e-12
    pooling: str = "mean"          # mean | cls
    position_offset: int = 0       # RoBERTa / XLM-R number positions from padding_idx + 1 (= 2)


def tiny_bert() -> BertConfig:
    return BertConfig(vocab_size=128, hidden=128, layers=2, heads=2, intermediate=256, max_len=32)


class BertEncoder:
    def __init__(self, cfg: BertConfig, device="cpu", get: Optional[Callable[[str], Optional[torch.Tensor]]] = None,
                 seed: int = 0, prefix: str = ""):
        self.cfg, self.device = cfg, torch.device(device)
        if get is not None and prefix == "" and get("embeddings.word_embeddings.weight") is None \
                and get("bert.embeddings.word_embeddings.weight") is not None:
            prefix = "bert."
        if get is not None and prefix == "" and get("embeddings.word_embeddings.weight") is None \
                and get("roberta.embeddings.word_embeddings.weight") is not None:
            prefix = "roberta."
        f = WeightFactory(self.device, False, get=get, seed=seed)
        H = cfg.hidden
        e = prefix + "embeddings."
        self.tok = f.tensor(e + "word_embeddings.weight", cfg.vocab_size, H)
        self.pos = f.tensor(e + "position_embeddings.weight", cfg.max_len, H)
        self.typ = f.tensor(e + "token_type_embeddings.weight", cfg.type_vocab, H)
        self.ln_w = f.tensor(e + "LayerNorm.weight", H, ones=True)
        self.ln_b = f.tensor(e + "LayerNorm.bias", H, zeros=True)
        self.blocks = []
        for i in range(cfg.layers):
            p = f"{prefix}encoder.layer.{i}."
            q, k, v = (f.linear(p + f"attention.self.{n}", H, H) for n in ("query", "key", "value"))
            self.blocks.append(dict(
                qkv=ops.LinearWeight(torch.cat([q.weight, k.weight, v.weight], 0), None, torch.cat([q.bias, k.bias, v.bias], 0)),
                o=f.linear(p + "attention.output.dense", H, H),
                ln1w=f.tensor(p + "attention.output.LayerNorm.weight", H, ones=True),
                ln1b=f.tensor(p + "attention.output.LayerNorm.bias", H, zeros=True),
                fc1=f.linear(p + "intermediate.dense", cfg.intermediate, H),
                fc2=f.linear(p + "output.dense", H, cfg.intermediate),
                ln2w=f.tensor(p + "output.LayerNorm.weight", H, ones=True),
                ln2b=f.tensor(p + "output.LayerNorm.bias", H, zeros=True)))

    @torch.no_grad()
    def hidden_states(self, ids: torch.Tensor, type_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
        """ids [L] (one unpadded sequence) -> [L, H]."""
        cfg = self.cfg
        L = ids.shape[0]
        off = cfg.position_offset
        if L + off > cfg.max_len:
            raise ValueError(f"sequence of {L} tokens exceeds the model's {cfg.max_len - off} positions")
        ids = ids.long().to(self.device)
        tt = torch.zeros_like(ids) if type_ids is None else type_ids.long().to(self.device)
        x = (self.tok[ids].float() + self.pos[off:off + L].float() + self.typ[tt].float()).to(torch.bfloat16)
        x, _, _ = ops.norm(x, self.ln_w, bias=self.ln_b, layernorm=True, eps=cfg.eps)
        d = cfg.hidden // cfg.heads
        for b in self.blocks:
            qkv = ops.linear(x, b["qkv"])
            q, k, v = ops.dit_qkv(qkv, cfg.heads, cfg.heads, d)
            a = ops.attention(q, k, v, causal=False)
            y = ops.linear(a.reshape(L, -1), b["o"], residual=x)
            x, _, _ = ops.norm(y, b["ln1w"], bias=b["ln1b"], layernorm=True, eps=cfg.eps)
            m = torch.nn.functional.gelu(ops.linear(x, b["fc1"]).float()).to(torch.bfloat16)
            y = ops.linear(m, b["fc2"], residual=x)
            x, _, _ = ops.norm(y, b["ln2w"], bias=b["ln2b"], layernorm=True, eps=cfg.eps)
        return x

    @torch.no_grad()
    def embed(self, ids: torch.Tensor, normalize: bool = True) -> torch.Tensor:
        h = self.hidden_states(ids).float()
        e = h[0] if self.cfg.pooling == "cls" else h.mean(dim=0)
        return torch.nn.functional.normalize(e, dim=0) if normalize else e
