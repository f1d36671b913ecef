"""Text-to-speech pipeline over a VITS checkpoint directory (``config.json``, weights, ``vocab.json``).

Text is normalised (lower-cased when the voice was trained that way, characters outside the
vocabulary dropped), mapped to character ids and, for voices trained with blanks, interleaved with
the blank id; long inputs are split at sentence punctuation and the pieces concatenated with a short
pause.

Reference: src/HartsyInference.Audio/Pipelines/PiperPipeline.cs, MeloTtsPipeline.cs (character /
phoneme id front end, sentence splitting), src/HartsyInference.Engine/Services/SpeechService.cs.
"""
from __future__ import annotations

import json
import re
from dataclasses import dataclass
from pathlib import Path
from typing import Optional

import torch

from ..models.audio.vits import VitsConfig, VitsModel, vits_from_hf


@dataclass
class SpeechResult:
    samples: torch.Tensor          # float32 [n] in [-1, 1]
    sample_rate: int
    seconds: float = 0.0


class VitsCharTokenizer:
    def __init__(self, vocab: dict[str, int], add_blank: bool = True, lower: bool = True, pad: str = "<pad>"):
        self.vocab, self.add_blank, self.lower = dict(vocab), add_blank, lower
        self.blank_id = self.vocab.get(pad, 0)

    @staticmethod
    def from_dir(path) -> "VitsCharTokenizer":
        p = Path(path)
        vocab = json.loads((p / "vocab.json").read_text(encoding="utf-8"))
        tc = json.loads((p / "tokenizer_config.json").read_text()) if (p / "tokenizer_config.json").exists() else {}
        return VitsCharTokenizer(vocab, bool(tc.get("add_blank", True)), bool(tc.get("normalize", True)), tc.get("pad_token", "<pad>"))

    def encode(self, text: str) -> list[int]:
        if self.lower:
            text = text.lower()
        ids = [self.vocab[c] for c in text if c in self.vocab]
        if self.add_blank:
            out = [self.blank_id] * (2 * len(ids) + 1)
            out[1::2] = ids
            return out
        return ids


_SPLIT = re.compile(r"(?<=[.!?;:。！？])\s+")


class VitsPipeline:
    def __init__(self, model: VitsModel, tokenizer: VitsCharTokenizer, max_chars: int = 300):
        self.model, self.tokenizer, self.max_chars = model, tokenizer, max_chars
        self.cfg: VitsConfig = model.cfg

    @staticmethod
    def from_pretrained(path, device="cuda") -> "VitsPipeline":
        from ..assets.safetensors import ShardedCheckpoint
        p = Path(path)
        raw = json.loads((p / "config.json").read_text())
        ck = ShardedCheckpoint(p)
        return VitsPipeline(VitsModel(vits_from_hf(raw), device, get=ck.get), VitsCharTokenizer.from_dir(p))

    def split(self, text: str) -> list[str]:
        """Sentences, packed into chunks of at most ``max_chars`` characters."""
        chunks: list[str] = []
        cur = ""
        for s in (t.strip() for t in _SPLIT.split(text.strip())):
            if not s:
                continue
            while len(s) > self.max_chars:                    # an over-long sentence is cut at a space
                cut = s.rfind(" ", 0, self.max_chars)
                cut = cut if cut > 0 else self.max_chars
                chunks.append((cur + " " + s[:cut]).strip() if cur else s[:cut])
                cur, s = "", s[cut:].strip()
            if cur and len(cur) + 1 + len(s) > self.max_chars:
                chunks.append(cur)
                cur = s
            else:
                cur = (cur + " " + s).strip()
        if cur:
            chunks.append(cur)
        return chunks

    @torch.no_grad()
    def speak(self, text: str, speaking_rate: Optional[float] = None, noise_scale: Optional[float] = None,
              noise_scale_duration: Optional[float] = None, pause_s: float = 0.15) -> SpeechResult:
        sr = self.cfg.sampling_rate
        pieces = []
        for chunk in self.split(text):
            ids = self.tokenizer.encode(chunk)
            if not ids or all(i == self.tokenizer.blank_id for i in ids):
                continue
            wav = self.model.synthesize(torch.tensor(ids), noise_scale, noise_scale_duration, speaking_rate)
            if pieces:
                pieces.append(torch.zeros(int(pause_s * sr)))
            pieces.append(wav.float().cpu())
        samples = torch.cat(pieces) if pieces else torch.zeros(0)
        return SpeechResult(samples, sr, samples.numel() / sr)
