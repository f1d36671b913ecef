"""Speech-to-text service: hosts Whisper pipelines by checkpoint path.

Reference: src/HartsyInference.Engine/Services/TranscribeService.cs, ITranscribeService.cs.
"""
from __future__ import annotations

import math
import threading
from pathlib import Path

import torch

from ..audio import read_wav
from ..pipelines.whisper import TranscriptResult, WhisperOptions, WhisperPipeline
from .requests import AudioRequest, ModelSpec


class _BarkVoice:
    """Bark checkpoint directory: weights, WordPiece tokenizer, ``generation_config.json`` (token bookkeeping of
    the three stages) and optional voice presets (``speaker_embeddings/<voice>_{semantic,coarse,fine}_prompt.npy``)."""

    def __init__(self, path: Path, raw: dict, device):
        import json
        from ..assets.safetensors import ShardedCheckpoint
        from ..assets.tokenizer import WordPieceTokenizer
        from ..models.audio.bark import Bark
        gen_file = path / "generation_config.json"
        generation = json.loads(gen_file.read_text()) if gen_file.exists() else {}
        dtype = torch.bfloat16 if str(device).startswith("cuda") else torch.float32
        self.path, self.model = path, Bark(raw, ShardedCheckpoint(path).get, device, dtype, generation)
        self.tokenizer = WordPieceTokenizer.from_dir(path)

    def _history(self, voice):
        if not voice:
            return None
        import numpy as np
        out = {}
        for part in ("semantic", "coarse", "fine"):
            hits = [self.path / "speaker_embeddings" / f"{voice}_{part}_prompt.npy", self.path / f"{voice}_{part}_prompt.npy"]
            f = next((h for h in hits if h.exists()), None)
            if f is None:
                raise ValueError(f"voice '{voice}': no {part} prompt beside the checkpoint")
            out[f"{part}_prompt"] = torch.from_numpy(np.load(f)).long()
        return out

    def speak(self, req):
        from ..pipelines.vits import SpeechResult
        ids = torch.tensor(self.tokenizer.encode(req.text, add_special=False) or [0])
        wave = self.model.generate(ids, self._history(req.voice), sample=not getattr(req, "greedy", False),
                                   seed=int(getattr(req, "seed", 0) or 0)).float().cpu().clamp(-1, 1)
        return SpeechResult(wave, self.model.sampling_rate, wave.numel() / self.model.sampling_rate)


class _CsmVoice:
    """CSM checkpoint directory (weights incl. the Mimi codec, ``tokenizer.json``). A turn is written
    ``<|begin_of_text|>[speaker]text<|end_of_text|>``; ``voice`` is the speaker number."""

    def __init__(self, path: Path, raw: dict, device):
        from ..assets.safetensors import ShardedCheckpoint
        from ..assets.tokenizer import Tokenizer
        from ..models.audio.csm import Csm
        dtype = torch.bfloat16 if str(device).startswith("cuda") else torch.float32
        self.model = Csm(raw, ShardedCheckpoint(path).get, device, dtype)
        self.tokenizer = Tokenizer.from_hf_json(path / "tokenizer.json")
        self.bos = raw.get("bos_token_id", 128000)
        self.eot = self.tokenizer.special_tokens.get("<|end_of_text|>")

    def speak(self, req):
        from ..pipelines.vits import SpeechResult
        body = self.tokenizer.encode(f"[{req.voice or 0}]{req.text}", add_special=False)
        ids = [self.bos] + body + ([self.eot] if self.eot is not None else [])
        limit = max(1, int(round(float(getattr(req, "max_seconds", 0) or 30.0) * self.model.codec.cfg.frame_rate)))
        wave = self.model.generate(torch.tensor(ids), max_frames=limit, sample=not getattr(req, "greedy", False),
                                   seed=int(getattr(req, "seed", 0) or 0)).float().cpu().clamp(-1, 1)
        return SpeechResult(wave, self.model.sampling_rate, wave.numel() / self.model.sampling_rate)


class _DiaVoice:
    """Dia checkpoint directory; the DAC codec it writes for sits in a ``dac`` (or ``audio_tokenizer``) subdirectory
    with its own ``config.json``. Text is read as bytes, the speaker tags ``[S1]`` / ``[S2]`` as bytes 1 / 2."""

    def __init__(self, path: Path, raw: dict, device):
        import json
        from ..assets.safetensors import ShardedCheckpoint
        from ..models.audio.dac import DacCodec, DacConfig
        from ..models.audio.dia import Dia
        dtype = torch.bfloat16 if str(device).startswith("cuda") else torch.float32
        sub = next((path / n for n in ("dac", "audio_tokenizer", "codec") if (path / n / "config.json").exists()), None)
        if sub is None:
            raise FileNotFoundError(f"{path}: no dac / audio_tokenizer subdirectory with the codec")
        codec_raw = json.loads((sub / "config.json").read_text())
        self.codec = DacCodec(DacConfig.from_hf(codec_raw), ShardedCheckpoint(sub).get, device)
        self.model = Dia(raw, ShardedCheckpoint(path).get, device, dtype, codec=self.codec)
        self.sampling_rate = codec_raw.get("sampling_rate", 44100)
        self.frame_rate = self.sampling_rate / self.codec.cfg.hop

    @staticmethod
    def text_bytes(text: str) -> list[int]:
        return list(text.replace("[S1]", "\x01").replace("[S2]", "\x02").encode("utf-8"))

    def speak(self, req):
        from ..pipelines.vits import SpeechResult
        text = req.text if req.text.lstrip().startswith("[S") else "[S1] " + req.text
        limit = max(2, int(round(float(getattr(req, "max_seconds", 0) or 30.0) * self.frame_rate))) + max(self.model.delays) + 2
        wave = self.model.generate(torch.tensor(self.text_bytes(text)), max_steps=limit, sample=not getattr(req, "greedy", False),
                                   temperature=1.3 if not getattr(req, "greedy", False) else 1.0,
                                   seed=int(getattr(req, "seed", 0) or 0)).float().cpu().clamp(-1, 1)
        return SpeechResult(wave, self.sampling_rate, wave.numel() / self.sampling_rate)


class SpeechService:
    """Text-to-speech: hosts VITS pipelines (MMS-TTS / Piper-class voices), Bark, CSM and Dia checkpoints by path.
    Reference: src/HartsyInference.Engine/Services/SpeechService.cs, ISpeechService.cs."""

    def __init__(self, device):
        self.device = device
        self._lock = threading.Lock()
        self._loaded: dict = {}

    def loaded_keys(self) -> list[str]:
        kind = lambda v: ("bark" if isinstance(v, _BarkVoice) else "csm" if isinstance(v, _CsmVoice) else
                          "dia" if isinstance(v, _DiaVoice) else "vits")
        return [f"{kind(v)}:{k}" for k, v in self._loaded.items()]

    def release(self) -> None:
        with self._lock:
            self._loaded.clear()

    def run(self, spec: ModelSpec, req):
        from ..pipelines.vits import VitsPipeline
        path = spec.local_path or spec.requested
        with self._lock:
            if path not in self._loaded:
                import json
                cfg_file = Path(path) / "config.json"
                raw = json.loads(cfg_file.read_text()) if cfg_file.exists() else {}
                if raw.get("model_type") == "bark":
                    self._loaded[path] = _BarkVoice(Path(path), raw, self.device)
                elif raw.get("model_type") == "csm":
                    self._loaded[path] = _CsmVoice(Path(path), raw, self.device)
                elif raw.get("model_type") == "dia":
                    self._loaded[path] = _DiaVoice(Path(path), raw, self.device)
                else:
                    self._loaded[path] = VitsPipeline.from_pretrained(path, self.device)
            pipe = self._loaded[path]
        if isinstance(pipe, (_BarkVoice, _CsmVoice, _DiaVoice)):
            return pipe.speak(req)
        return pipe.speak(req.text, speaking_rate=req.speed, noise_scale=req.noise_scale,
                          noise_scale_duration=req.noise_scale_duration)


class MusicService:
    """Text-to-music: hosts MusicGen checkpoints (T5 text encoder, codebook language model, EnCodec
    decoder in one directory) by path. Reference: src/HartsyInference.Engine/Services (music)."""

    def __init__(self, device):
        self.device = device
        self._lock = threading.Lock()
        self._loaded: dict = {}

    def loaded_keys(self) -> list[str]:
        return [f"musicgen:{k}" for k in self._loaded]

    def release(self) -> None:
        with self._lock:
            self._loaded.clear()

    def run(self, spec: ModelSpec, req):
        import json
        from pathlib import Path
        from ..assets.safetensors import ShardedCheckpoint
        from ..assets.tokenizer import ByteTokenizer, UnigramTokenizer
        from ..models.audio.musicgen import Musicgen
        from ..pipelines.vits import SpeechResult
        path = Path(spec.local_path or spec.requested)
        with self._lock:
            if str(path) not in self._loaded:
                raw = json.loads((path / "config.json").read_text())
                model = Musicgen(raw, ShardedCheckpoint(path).get, self.device)
                tok = (UnigramTokenizer.from_hf_json(path / "tokenizer.json") if (path / "tokenizer.json").exists()
                       else ByteTokenizer(vocab_size=raw["text_encoder"]["vocab_size"]))
                self._loaded[str(path)] = (model, tok, raw)
            model, tok, raw = self._loaded[str(path)]
        ids = tok.encode(req.prompt)
        ids = [i for i in ids if i < raw["text_encoder"]["vocab_size"]] or [0]
        frame_rate = model.sampling_rate / math.prod(model.codec.cfg.ratios)
        frames = max(1, int(round(req.seconds * frame_rate)))
        wave = model.generate(torch.tensor(ids), frames, guidance=req.guidance, sample=not req.greedy, seed=req.seed)
        samples = wave.mean(0).float().cpu().clamp(-1, 1)
        return SpeechResult(samples, model.sampling_rate, samples.numel() / model.sampling_rate)


class _KyutaiTranscriber:
    """Kyutai speech-to-text checkpoint directory (language model + Mimi codec, ``tokenizer.json`` or
    ``tokenizer.model``-derived json). Words come out ``audio_delay_seconds`` after they were spoken; a segment is
    written per word run with the time of the frame that produced its first piece, shifted back by the delay."""

    def __init__(self, path: Path, raw: dict, device):
        import json
        from ..assets.safetensors import ShardedCheckpoint
        from ..assets.tokenizer import Tokenizer
        from ..models.audio.kyutai_stt import KyutaiStt
        dtype = torch.bfloat16 if str(device).startswith("cuda") else torch.float32
        self.model = KyutaiStt(raw, ShardedCheckpoint(path).get, device, dtype)
        self.tokenizer = Tokenizer.from_hf_json(path / "tokenizer.json")
        pre = path / "preprocessor_config.json"
        extra = json.loads(pre.read_text()) if pre.exists() else {}
        self.delay = float(extra.get("audio_delay_seconds", 2.5))
        self.prefix = float(extra.get("audio_silence_prefix_seconds", 1.0))

    def transcribe(self, audio: torch.Tensor, rate: int, opts) -> TranscriptResult:
        from ..audio.wav import resample
        from ..pipelines.whisper import WhisperSegment
        x = audio.float()
        x = x.mean(0) if x.dim() > 1 else x
        want = self.model.codec.cfg.sampling_rate
        if rate != want:
            x = resample(x, rate, want)
        tokens = self.model.transcribe_tokens(x, self.delay, self.prefix)
        frame = self.model.cfg.frame_size / want
        skip = {self.model.cfg.pad, self.model.cfg.bos}
        segments, run, start = [], [], 0.0
        for i, t in enumerate(tokens.tolist() + [self.model.cfg.pad]):
            if t in skip:
                if run:
                    text = self.tokenizer.decode(run)
                    end = max(i * frame - self.delay - self.prefix, start)
                    segments.append(WhisperSegment(start=start, end=end, text=text, tokens=list(run)))
                    run = []
                continue
            if not run:
                start = max(i * frame - self.delay - self.prefix, 0.0)
            run.append(t)
        text = " ".join(s.text.strip() for s in segments if s.text.strip())
        return TranscriptResult(text=text, language=None, segments=segments, duration_s=x.numel() / want)


class TranscribeService:
    def __init__(self, device):
        self.device = device
        self._lock = threading.Lock()
        self._loaded: dict[str, WhisperPipeline] = {}

    def loaded_keys(self) -> list[str]:
        return [f"{'kyutai' if isinstance(v, _KyutaiTranscriber) else 'whisper'}:{k}" for k, v in self._loaded.items()]

    def release(self) -> None:
        with self._lock:
            self._loaded.clear()

    def _pipe(self, spec: ModelSpec) -> WhisperPipeline:
        path = spec.local_path or spec.requested
        with self._lock:
            if path not in self._loaded:
                import json
                from ..pipelines.whisper import MoonshinePipeline
                cfg_file = Path(path) / "config.json"
                kind = json.loads(cfg_file.read_text()).get("model_type", "whisper") if cfg_file.exists() else "whisper"
                if kind == "kyutai_speech_to_text":
                    self._loaded[path] = _KyutaiTranscriber(Path(path), json.loads(cfg_file.read_text()), self.device)
                else:
                    cls = MoonshinePipeline if kind == "moonshine" else WhisperPipeline
                    self._loaded[path] = cls.from_pretrained(path, self.device)
            return self._loaded[path]

    def run(self, spec: ModelSpec, req: AudioRequest) -> TranscriptResult:
        a, rate = req.audio, req.sample_rate
        if isinstance(a, (str, Path, bytes, bytearray)):
            a, rate = read_wav(a)
        if a is None:
            raise ValueError("AudioRequest.audio is empty")
        opts = WhisperOptions(language=req.language, task=req.task, timestamps=req.timestamps)
        with self._lock:
            pipe = self._loaded.get(spec.local_path or spec.requested)
        pipe = pipe or self._pipe(spec)
        return pipe.transcribe(torch.as_tensor(a), rate, opts)
