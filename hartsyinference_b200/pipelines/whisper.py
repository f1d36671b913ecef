"""Whisper speech recognition: log-mel front end, 30-second windows that advance by the last
timestamp the decoder emitted, language detection, greedy decoding under the timestamp grammar,
segments with start / end times.

Reference: src/HartsyInference.Audio/Pipelines/WhisperPipeline.cs, WhisperOptions.cs,
WhisperSegment.cs; src/HartsyInference.Engine/Services/TranscribeService.cs.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Optional

import torch

from ..audio import log_mel_spectrogram, resample
from ..models.audio.whisper import WhisperConfig, WhisperModel, whisper_from_hf

SAMPLE_RATE = 16000
HOP = 160
TIME_PER_TOKEN = 0.02          # one timestamp token = two mel frames after the stride-2 convolution


@dataclass
class WhisperSegment:
    start: float
    end: float
    text: str
    tokens: list[int] = field(default_factory=list)
    avg_logprob: float = 0.0
    no_speech_prob: float = 0.0


@dataclass
class TranscriptResult:
    text: str = ""
    language: Optional[str] = None
    segments: list[WhisperSegment] = field(default_factory=list)
    duration_s: float = 0.0


@dataclass
class WhisperOptions:
    language: Optional[str] = None          # None = detect (multilingual checkpoints)
    task: str = "transcribe"                # or "translate"
    timestamps: bool = True
    max_initial_timestamp: float = 1.0
    no_speech_threshold: float = 0.6
    logprob_threshold: float = -1.0
    max_new_tokens: int = 0                 # 0 = the decoder's context


@dataclass
class WhisperVocab:
    """Ids of the control tokens. ``timestamp_begin`` is the id of <|0.00|>."""
    sot: int
    eot: int
    transcribe: int
    translate: int
    no_timestamps: int
    timestamp_begin: int
    no_speech: int = -1
    languages: dict[str, int] = field(default_factory=dict)
    suppress: list[int] = field(default_factory=list)
    begin_suppress: list[int] = field(default_factory=list)

    @staticmethod
    def from_special_tokens(specials: dict[str, int], suppress=(), begin_suppress=()) -> "WhisperVocab":
        def need(*names):
            for n in names:
                if n in specials:
                    return specials[n]
            raise KeyError(names[0])
        nots = need("<|notimestamps|>")
        langs = {k[2:-2]: v for k, v in specials.items()
                 if k.startswith("<|") and k.endswith("|>") and 2 <= len(k) - 4 <= 3 and k[2:-2].isalpha() and k[2:-2].islower()}
        return WhisperVocab(sot=need("<|startoftranscript|>"), eot=need("<|endoftext|>"), transcribe=need("<|transcribe|>"),
                            translate=need("<|translate|>"), no_timestamps=nots, timestamp_begin=nots + 1,
                            no_speech=specials.get("<|nospeech|>", specials.get("<|nocaptions|>", -1)),
                            languages=langs, suppress=list(suppress or ()), begin_suppress=list(begin_suppress or ()))


class WhisperPipeline:
    def __init__(self, model: WhisperModel, vocab: WhisperVocab, tokenizer=None):
        self.model, self.vocab, self.tokenizer = model, vocab, tokenizer
        self.cfg: WhisperConfig = model.cfg
        self.window_frames = self.cfg.max_source * 2              # mel frames one encoder pass covers
        self.window_samples = self.window_frames * HOP

    @staticmethod
    def from_pretrained(path, device="cuda") -> "WhisperPipeline":
        from ..assets.safetensors import ShardedCheckpoint
        from ..assets.tokenizer import Tokenizer
        p = Path(path)
        raw = json.loads((p / "config.json").read_text())
        ck = ShardedCheckpoint(p)
        model = WhisperModel(whisper_from_hf(raw), device, get=ck.get)
        tok = Tokenizer.from_hf_json(p / "tokenizer.json")
        gen = json.loads((p / "generation_config.json").read_text()) if (p / "generation_config.json").exists() else {}
        vocab = WhisperVocab.from_special_tokens(tok.special_tokens, gen.get("suppress_tokens", raw.get("suppress_tokens")),
                                                 gen.get("begin_suppress_tokens", raw.get("begin_suppress_tokens")))
        return WhisperPipeline(model, vocab, tok)

    # ------------------------------------------------------------------------------ decoding rules
    def _mask_logits(self, logits: torch.Tensor, seq: list[int], prompt_len: int, opts: WhisperOptions) -> torch.Tensor:
        """The decoder's grammar, applied to the logits of the next token (in place)."""
        v = self.vocab
        ninf = float("-inf")
        if v.suppress:
            logits[v.suppress] = ninf
        logits[[v.sot, v.transcribe, v.translate]] = ninf
        if v.no_speech >= 0:
            logits[v.no_speech] = ninf
        for lid in v.languages.values():
            logits[lid] = ninf
        sampled = seq[prompt_len:]
        if not sampled and v.begin_suppress:
            logits[v.begin_suppress] = ninf
        if not sampled:
            logits[v.eot] = ninf                       # nothing decoded yet: an empty segment is decided by no-speech
        if not opts.timestamps:
            logits[v.timestamp_begin:] = ninf
            return logits
        logits[v.no_timestamps] = ninf
        tb = v.timestamp_begin
        last_ts = bool(sampled) and sampled[-1] >= tb
        prev_ts = len(sampled) < 2 or sampled[-2] >= tb
        if last_ts:
            if prev_ts:
                logits[tb:] = ninf                     # a pair just closed (or opened at the start): text next
            else:
                logits[: v.eot] = ninf                 # text ended with one timestamp: its pair or the end
        stamps = [t for t in sampled if t >= tb]
        if stamps:
            floor = stamps[-1] if (last_ts and not prev_ts) else stamps[-1] + 1
            logits[tb:floor] = ninf                    # timestamps never go backwards
        if not sampled:
            logits[:tb] = ninf                         # a window opens with a timestamp
            last = tb + int(round(opts.max_initial_timestamp / TIME_PER_TOKEN))
            logits[last + 1:] = ninf
        lp = torch.log_softmax(logits.float(), -1)
        if torch.logsumexp(lp[tb:], -1) > lp[:tb].max():
            logits[:tb] = ninf                         # timestamps together outweigh every text token
        return logits

    @torch.no_grad()
    def detect_language(self, enc: torch.Tensor) -> tuple[Optional[str], dict[str, float]]:
        v = self.vocab
        if not v.languages:
            return None, {}
        st = self.model.start(enc)
        logits = self.model.decode(st, torch.tensor([v.sot], dtype=torch.int32))[0]
        ids = torch.tensor(list(v.languages.values()))
        probs = torch.softmax(logits[ids.to(logits.device)].float(), -1).cpu()
        names = list(v.languages)
        best = names[int(probs.argmax())]
        return best, {n: float(p) for n, p in zip(names, probs)}

    @torch.no_grad()
    def _decode_window(self, enc: torch.Tensor, language: Optional[str], opts: WhisperOptions):
        v = self.vocab
        prompt = [v.sot]
        if language is not None and language in v.languages:
            prompt.append(v.languages[language])
        if v.languages:
            prompt.append(v.translate if opts.task == "translate" else v.transcribe)
        if not opts.timestamps:
            prompt.append(v.no_timestamps)
        st = self.model.start(enc)
        logits = self.model.decode(st, torch.tensor(prompt, dtype=torch.int32))
        no_speech = 0.0
        if v.no_speech >= 0:
            no_speech = float(torch.softmax(logits[0].float(), -1)[v.no_speech])
        seq = list(prompt)
        limit = self.cfg.max_target - len(prompt) - 1
        if opts.max_new_tokens:
            limit = min(limit, opts.max_new_tokens)
        nxt = logits[-1]
        total_lp, n_lp = 0.0, 0
        for _ in range(max(limit, 0)):
            raw_lp = torch.log_softmax(nxt.float(), -1)
            masked = self._mask_logits(nxt.clone(), seq, len(prompt), opts)
            tok = int(masked.argmax())
            total_lp += float(raw_lp[tok])
            n_lp += 1
            if tok == v.eot:
                break
            seq.append(tok)
            nxt = self.model.decode(st, torch.tensor([tok], dtype=torch.int32))[0]
        return seq[len(prompt):], (total_lp / max(n_lp, 1)), no_speech

    def _text(self, tokens: list[int]) -> str:
        toks = [t for t in tokens if t < self.vocab.eot]
        if self.tokenizer is None:
            return " ".join(str(t) for t in toks)
        return self.tokenizer.decode(toks)

    def _segments(self, tokens: list[int], offset_s: float, window_s: float, avg_lp: float, no_speech: float):
        """Split one window's tokens at timestamp pairs. Returns (segments, seconds to advance)."""
        tb = self.vocab.timestamp_begin
        is_ts = [t >= tb for t in tokens]
        segs: list[WhisperSegment] = []
        pairs = [i for i in range(1, len(tokens)) if is_ts[i] and is_ts[i - 1]]
        ends_single = len(tokens) >= 2 and is_ts[-1] and not is_ts[-2]
        if pairs:
            cut = pairs + ([len(tokens)] if ends_single else [])
            last = 0
            for c in cut:
                sl = tokens[last:c]
                stamps = [t for t in sl if t >= tb]
                if stamps:
                    s0, s1 = (stamps[0] - tb) * TIME_PER_TOKEN, (stamps[-1] - tb) * TIME_PER_TOKEN
                    segs.append(WhisperSegment(offset_s + s0, offset_s + s1, self._text(sl), [t for t in sl if t < tb], avg_lp, no_speech))
                last = c
            if ends_single:
                advance = window_s                     # the window's speech was closed by a lone end stamp
            else:
                advance = (tokens[last - 1] - tb) * TIME_PER_TOKEN
        else:
            stamps = [t for t in tokens if t >= tb]
            end = (stamps[-1] - tb) * TIME_PER_TOKEN if stamps and stamps[-1] != tb else window_s
            start = (stamps[0] - tb) * TIME_PER_TOKEN if stamps else 0.0
            if any(not f for f in is_ts):
                segs.append(WhisperSegment(offset_s + start, offset_s + end, self._text(tokens), [t for t in tokens if t < tb], avg_lp, no_speech))
            advance = window_s
        return segs, advance

    # ------------------------------------------------------------------------------ public
    @torch.no_grad()
    def transcribe(self, audio: torch.Tensor, rate: int = SAMPLE_RATE, options: Optional[WhisperOptions] = None) -> TranscriptResult:
        """audio [n] or [channels, n] float in [-1, 1] at ``rate`` Hz."""
        opts = options or WhisperOptions()
        x = audio.float()
        if x.ndim == 2:
            x = x.mean(0)
        x = resample(x, rate, SAMPLE_RATE)
        total = x.numel()
        window_s = self.window_samples / SAMPLE_RATE
        res = TranscriptResult(duration_s=total / SAMPLE_RATE, language=opts.language)
        seek = 0
        while seek < total:
            chunk = x[seek: seek + self.window_samples]
            if chunk.numel() < HOP * 2:
                break
            mel = log_mel_spectrogram(chunk, self.cfg.n_mels, SAMPLE_RATE, chunk_seconds=window_s)
            enc = self.model.encode(mel)
            if res.language is None and self.vocab.languages:
                res.language, _ = self.detect_language(enc)
            tokens, avg_lp, no_speech = self._decode_window(enc, res.language, opts)
            span_s = min(window_s, (total - seek) / SAMPLE_RATE)
            if no_speech > opts.no_speech_threshold and avg_lp < opts.logprob_threshold:
                seek += self.window_samples
                continue
            if opts.timestamps:
                segs, advance = self._segments(tokens, seek / SAMPLE_RATE, span_s, avg_lp, no_speech)
            else:
                segs = [WhisperSegment(seek / SAMPLE_RATE, seek / SAMPLE_RATE + span_s, self._text(tokens), list(tokens), avg_lp, no_speech)]
                advance = window_s
            res.segments += [s for s in segs if s.text.strip() or s.tokens]
            seek += max(int(round(advance * SAMPLE_RATE)), HOP * 2)
        res.text = "".join(s.text for s in res.segments).strip() if self.tokenizer is not None else " ".join(s.text for s in res.segments)
        return res


class MoonshinePipeline:
    """Moonshine speech recognition over raw audio: resample to 16 kHz, cut long recordings into
    windows at the quietest point near each boundary, greedy-decode each window.
    Reference: src/HartsyInference.Audio/Pipelines/MoonshinePipeline.cs, MoonshineOptions.cs."""

    def __init__(self, model, tokenizer=None, window_s: float = 30.0):
        self.model, self.tokenizer, self.window_s = model, tokenizer, window_s

    @staticmethod
    def from_pretrained(path, device="cuda") -> "MoonshinePipeline":
        from ..assets.safetensors import ShardedCheckpoint
        from ..assets.tokenizer import Tokenizer
        from ..models.audio.moonshine import MoonshineModel, moonshine_from_hf
        p = Path(path)
        raw = json.loads((p / "config.json").read_text())
        tok = Tokenizer.from_hf_json(p / "tokenizer.json") if (p / "tokenizer.json").exists() else None
        return MoonshinePipeline(MoonshineModel(moonshine_from_hf(raw), device, get=ShardedCheckpoint(p).get), tok)

    def _windows(self, x: torch.Tensor) -> list[tuple[int, int]]:
        n, w = x.numel(), int(self.window_s * SAMPLE_RATE)
        out, start = [], 0
        while n - start > w:
            lo = start + int(0.8 * w)                      # look for a quiet 20 ms frame in the window's last fifth
            frames = x[lo:start + w].abs().unfold(0, 320, 320).mean(-1)
            cut = lo + int(frames.argmin()) * 320 + 160
            out.append((start, cut))
            start = cut
        out.append((start, n))
        return out

    @torch.no_grad()
    def transcribe(self, audio: torch.Tensor, rate: int = SAMPLE_RATE, options: Optional[WhisperOptions] = None) -> TranscriptResult:
        x = audio.float()
        if x.ndim == 2:
            x = x.mean(0)
        x = resample(x, rate, SAMPLE_RATE)
        res = TranscriptResult(duration_s=x.numel() / SAMPLE_RATE, language="en")
        for a, b in self._windows(x):
            if b - a < 1024:                                # shorter than the first convolution's reach
                continue
            toks = self.model.transcribe_tokens(x[a:b], (options.max_new_tokens or None) if options else None)
            text = self.tokenizer.decode(toks) if self.tokenizer is not None else " ".join(str(t) for t in toks)
            res.segments.append(WhisperSegment(a / SAMPLE_RATE, b / SAMPLE_RATE, text, toks))
        res.text = " ".join(s.text.strip() for s in res.segments).strip()
        return res


class StreamingTranscriber:
    """Incremental transcription of a live audio stream. Audio is pushed in pieces of any size; each
    push transcribes the not-yet-committed audio and returns (committed segments that are new, the
    current tentative text). A segment is committed once it ends at least ``hold_s`` before the end
    of the audio received so far, so late context can still revise the tail; ``flush`` commits the rest.

    Reference: src/HartsyInference.Audio/Pipelines/WhisperStreamingPipeline.cs, MoonshineStreamingPipeline.cs."""

    def __init__(self, pipeline, rate: int = SAMPLE_RATE, hold_s: float = 2.0, options: Optional[WhisperOptions] = None):
        self.pipe, self.rate, self.hold_s, self.options = pipeline, rate, hold_s, options
        self.buffer = torch.zeros(0)
        self.offset_s = 0.0                      # stream time of buffer[0]
        self.committed: list[WhisperSegment] = []

    def push(self, samples: torch.Tensor) -> tuple[list[WhisperSegment], str]:
        x = samples.float()
        if x.ndim == 2:
            x = x.mean(0)
        self.buffer = torch.cat([self.buffer, resample(x, self.rate, SAMPLE_RATE)])
        return self._advance(final=False)

    def flush(self) -> tuple[list[WhisperSegment], str]:
        return self._advance(final=True)

    def _advance(self, final: bool) -> tuple[list[WhisperSegment], str]:
        have_s = self.buffer.numel() / SAMPLE_RATE
        if have_s < 0.2:
            return [], ""
        res = self.pipe.transcribe(self.buffer, SAMPLE_RATE, self.options)
        new: list[WhisperSegment] = []
        tentative: list[str] = []
        cut_s = 0.0
        for seg in res.segments:
            if final or seg.end <= have_s - self.hold_s:
                new.append(WhisperSegment(seg.start + self.offset_s, seg.end + self.offset_s, seg.text, seg.tokens,
                                          seg.avg_logprob, seg.no_speech_prob))
                cut_s = max(cut_s, seg.end)
            else:
                tentative.append(seg.text)
        if final:
            cut_s = have_s
        if cut_s > 0:
            n = min(int(round(cut_s * SAMPLE_RATE)), self.buffer.numel())
            self.buffer = self.buffer[n:]
            self.offset_s += n / SAMPLE_RATE
        self.committed += new
        return new, "".join(tentative).strip()

    @property
    def text(self) -> str:
        return "".join(s.text for s in self.committed).strip()
