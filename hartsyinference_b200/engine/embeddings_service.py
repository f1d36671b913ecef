"""Sentence embeddings from encoder checkpoints (BERT family). Decoder checkpoints keep going
through ``TextService.embed`` (mean-pooled final hidden states).

Reference: src/HartsyInference.LLM/Embeddings/BertEmbeddingModel.cs, the ``/v1/embeddings`` route
(src/HartsyInference.Api/Endpoints/CompatEndpoints.cs:133).
"""
from __future__ import annotations

import json
import threading
from pathlib import Path

import torch

from ..assets.safetensors import ShardedCheckpoint
from ..assets.tokenizer import WordPieceTokenizer
from ..models.encoders.bert import BertConfig, BertEncoder
from .requests import ModelSpec


def is_bert_dir(path) -> bool:
    cfg = Path(path) / "config.json" if path else None
    if cfg is None or not cfg.exists():
        return False
    try:
        return json.loads(cfg.read_text()).get("model_type") in ("bert", "roberta", "xlm-roberta")
    except Exception:
        return False


class _FramedUnigram:
    """Unigram tokenizer with RoBERTa framing: ``<s> pieces </s>``."""

    def __init__(self, path, bos_id: int, eos_id: int):
        from ..assets.tokenizer import UnigramTokenizer
        self.tok, self.bos_id, self.eos_id = UnigramTokenizer.from_hf_json(path), bos_id, eos_id

    def encode(self, text: str) -> list[int]:
        return [self.bos_id] + self.tok.encode(text, add_special=False) + [self.eos_id]


class BertEmbeddingsService:
    def __init__(self, device):
        self.device = device
        self._lock = threading.Lock()
        self._loaded: dict[str, tuple[BertEncoder, WordPieceTokenizer]] = {}

    def _load(self, path: str):
        with self._lock:
            if path not in self._loaded:
                d = json.loads((Path(path) / "config.json").read_text())
                pooling = "mean"
                pool_cfg = Path(path) / "1_Pooling" / "config.json"
                if pool_cfg.exists() and json.loads(pool_cfg.read_text()).get("pooling_mode_cls_token"):
                    pooling = "cls"
                roberta = d.get("model_type") in ("roberta", "xlm-roberta")
                cfg = BertConfig(vocab_size=d["vocab_size"], hidden=d["hidden_size"], layers=d["num_hidden_layers"],
                                 heads=d["num_attention_heads"], intermediate=d["intermediate_size"],
                                 max_len=d.get("max_position_embeddings", 512), type_vocab=d.get("type_vocab_size", 2),
                                 eps=d.get("layer_norm_eps", 1e-12), pooling=pooling,
                                 position_offset=(d.get("pad_token_id", 1) + 1) if roberta else 0)
                ck = ShardedCheckpoint(path)
                enc = BertEncoder(cfg, self.device, get=ck.get)
                if roberta:      # XLM-R / multilingual-E5 / BGE-M3 class: SentencePiece unigram, <s> ... </s> framing
                    self._loaded[path] = (enc, _FramedUnigram(Path(path) / "tokenizer.json", d.get("bos_token_id", 0), d.get("eos_token_id", 2)))
                else:
                    self._loaded[path] = (enc, WordPieceTokenizer.from_dir(path))
            return self._loaded[path]

    def embed(self, spec: ModelSpec, texts: list[str]) -> torch.Tensor:
        enc, tok = self._load(spec.local_path or spec.requested)
        outs = []
        for t in texts:
            ids = tok.encode(t)[: enc.cfg.max_len]
            outs.append(enc.embed(torch.tensor(ids)).float().cpu())
        return torch.stack(outs)
