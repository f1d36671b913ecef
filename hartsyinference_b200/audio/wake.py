"""Wake-word detection: PCM in, detections out, one score every 80 ms.

The chain is the openWakeWord one, so its published weights load as they are:

* :class:`WakeMel` - 32-bin mel front end. The STFT is a stored DFT basis applied as a strided
  convolution (257 real + 257 imaginary filters of length 512, hop 160, no centring), power
  spectrum, mel projection, ``10 log10``, a floor at (maximum of the buffer - 80 dB), then
  ``x / 10 + 2``. Samples are in int16 scale (about +-32768). ``ceil(n / 160 - 3)`` frames.
* :class:`SpeechEmbedding` - frozen backbone shared by every wake word: a 76 x 32 mel window
  (about 775 ms) -> one 96-d vector. Nineteen convolutions alternating ``1 x 3`` over frequency
  (padded) and ``3 x 1`` over time (unpadded), channels 24 -> 48 -> 72 -> 96, max-pools between
  the stages, BatchNorm already folded, activation ``max(leaky_relu(x, 0.2), -0.4)``; a last
  bias-free ``3 x 1`` convolution collapses the remaining three time steps.
* :class:`WakeHead` - one wake word: 16 consecutive embeddings (1.28 s) flattened to 1536 ->
  hidden layers (each Linear, optional LayerNorm, ReLU) -> one sigmoid. The layout is read off the
  weight names (``nn.Sequential`` indices, optional ``model.`` prefix; rank-2 weight = Linear,
  rank-1 = LayerNorm; ``verifier_model.*`` ignored), so heads with and without LayerNorm load.
* :class:`WakeHeadTrainer` - trains a head (1536 -> H -> H -> 1, no LayerNorm) on feature windows
  with Adam and a positive-class weight, and exports it under the names :class:`WakeHead` reads.
* :class:`SileroVad` - voice-activity gate: 512-sample chunks at +-1 scale (+ 64 samples of carried
  context, reflect-padded to 640), DFT-basis convolution (258 filters of 256, hop 128) ->
  magnitude -> four ReLU convolutions (strides 1, 2, 2, 1) that leave one frame -> one LSTM cell
  step -> ReLU -> 1 x 1 convolution -> sigmoid.
* :class:`WakeDetector` - the streaming contract: every 1280 new samples the mel of those samples
  plus 480 samples of left context is computed (exactly 8 frames, because the dB floor is a
  reduction over the buffer it is given), appended to a mel ring; the newest 76 frames are embedded,
  the newest 16 embeddings scored by every head; a word fires when the mean of its last
  ``smoothing`` scores reaches its threshold, then stays quiet for ``refractory`` seconds. Nothing
  is scored before 76 real mel frames and 16 real embeddings exist.

Many streams can share one set of models: every model call here takes a batch, and
:func:`features_for_clips` pushes whole training sets through the same code path on the device.

Reference: src/HartsyInference.Audio/Models/Wake/ (WakeMelFrontend, SpeechEmbeddingModel, WakeHead,
WakeHeadTrainer, SileroVad, SileroVadStream), Pipelines/WakeDetectionPipeline.cs.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from pathlib import Path
from typing import Callable, Iterable, Optional

import torch
import torch.nn.functional as F

from .dsp import hann_window, mel_filterbank

RATE = 16000
HOP, N_FFT, MEL_BINS = 160, 512, 32
WINDOW_FRAMES, STRIDE_FRAMES, EMBED_DIM = 76, 8, 96
HEAD_FRAMES = 16
CHUNK = 1280
LEFT_CONTEXT = 3 * HOP


def load_tensors(path) -> dict:
    """Initializers of an ``.onnx`` file, or the tensors of a ``.safetensors`` file."""
    p = Path(path)
    if p.suffix == ".onnx":
        from ..assets.onnx_reader import read_onnx_initializers
        return read_onnx_initializers(p)
    from ..assets.safetensors import SafeTensorsFile
    f = SafeTensorsFile(p)
    return {k: f.get(k) for k in f.keys()}


def dft_basis(n_fft: int, window: Optional[torch.Tensor] = None) -> tuple[torch.Tensor, torch.Tensor]:
    """(real, imaginary) filters [n_fft / 2 + 1, 1, n_fft] of a windowed DFT."""
    k = torch.arange(n_fft // 2 + 1, dtype=torch.float64)[:, None]
    n = torch.arange(n_fft, dtype=torch.float64)[None]
    ang = 2 * math.pi * k * n / n_fft
    w = (window if window is not None else hann_window(n_fft)).double()[None]
    return (ang.cos() * w).float()[:, None], (-ang.sin() * w).float()[:, None]


class WakeMel:
    def __init__(self, weights: Optional[dict] = None, device="cpu"):
        self.device = torch.device(device)
        if weights is None:                        # the transform stated analytically (Hann window, Slaney mel scale)
            real, imag = dft_basis(N_FFT)
            mel = mel_filterbank(MEL_BINS, N_FFT, RATE, 60.0, 3800.0).t().contiguous()
        else:
            real, imag, mel = (weights[k].float() for k in ("0.stft.conv_real.weight", "0.stft.conv_imag.weight", "1.melW"))
        if tuple(real.shape) != (N_FFT // 2 + 1, 1, N_FFT) or tuple(mel.shape) != (N_FFT // 2 + 1, MEL_BINS):
            raise ValueError(f"wake mel: basis {tuple(real.shape)} / filterbank {tuple(mel.shape)} do not match 257 x 512 / 257 x 32")
        self.basis = torch.cat([real, imag], 0).to(self.device)
        self.mel = mel.to(self.device)

    @staticmethod
    def frame_count(samples: int) -> int:
        return max(0, math.ceil(samples / HOP - 3))

    @torch.no_grad()
    def __call__(self, samples: torch.Tensor) -> torch.Tensor:
        """samples [B, n] or [n] (int16 scale) -> mel [B, frames, 32]; the dB floor is taken per row."""
        x = samples.to(self.device).float()
        if x.dim() == 1:
            x = x[None]
        frames = self.frame_count(x.shape[-1])
        if frames <= 0:
            raise ValueError(f"wake mel needs at least {4 * HOP} samples, got {x.shape[-1]}")
        spec = F.conv1d(x[:, None], self.basis, stride=HOP)[:, :, :frames]
        half = self.basis.shape[0] // 2
        power = spec[:, :half] ** 2 + spec[:, half:] ** 2
        db = 10.0 * torch.log10((power.transpose(1, 2) @ self.mel).clamp_min(1e-10))
        floor = db.amax((1, 2), keepdim=True) - 80.0
        return torch.maximum(db, floor) / 10.0 + 2.0


_CONVS = [(3, 3, 0, 1), (1, 3, 0, 1), (3, 1, 0, 0)] + [(1, 3, 0, 1), (3, 1, 0, 0)] * 8
_POOLS = {2: (2, 2), 6: (1, 2), 10: (2, 2), 14: (1, 2), 18: (2, 2)}
_WIDTHS = [24] * 3 + [24] * 4 + [48] * 4 + [72] * 4 + [96] * 4


class SpeechEmbedding:
    def __init__(self, weights: Optional[dict] = None, device="cpu", seed: int = 0):
        self.device = torch.device(device)
        self.convs = []
        if weights is None:                        # random weights of the right shapes (tests, dry runs)
            g, cin = torch.Generator().manual_seed(seed), 1
            for (kh, kw, _, _), co in zip(_CONVS, _WIDTHS):
                self.convs.append((torch.randn(co, cin, kh, kw, generator=g) * (2.0 / (cin * kh * kw)) ** 0.5, torch.zeros(co)))
                cin = co
            self.final = torch.randn(EMBED_DIM, cin, 3, 1, generator=g) * (1.0 / (3 * cin)) ** 0.5
        else:
            for i in range(len(_CONVS)):
                name = "model/conv2d/Conv2D" if i == 0 else f"model/conv2d_{i}/Conv2D"
                self.convs.append((weights[name + "_weights_fused_bn"].float(), weights[name + "_bias_fused_bn"].float()))
            self.final = weights["model/conv2d_19/Conv2D/ReadVariableOp:0"].float()
        self.convs = [(w.to(self.device), b.to(self.device)) for w, b in self.convs]
        self.final = self.final.to(self.device)

    @torch.no_grad()
    def __call__(self, mel: torch.Tensor) -> torch.Tensor:
        """mel windows [B, 76, 32] -> embeddings [B, 96]."""
        if mel.shape[-2:] != (WINDOW_FRAMES, MEL_BINS):
            raise ValueError(f"embedding window must be {WINDOW_FRAMES} x {MEL_BINS}, got {tuple(mel.shape[-2:])}")
        x = mel.to(self.device).float().reshape(-1, 1, WINDOW_FRAMES, MEL_BINS)
        for i, ((kh, kw, ph, pw), (w, b)) in enumerate(zip(_CONVS, self.convs)):
            x = F.conv2d(x, w, b, padding=(ph, pw))
            x = F.leaky_relu(x, 0.2).clamp_min(-0.4)
            if i in _POOLS:
                x = F.max_pool2d(x, _POOLS[i], _POOLS[i])
        x = F.conv2d(x, self.final)
        if x.shape[1:] != (EMBED_DIM, 1, 1):
            raise RuntimeError(f"speech embedding backbone produced {tuple(x.shape)}")
        return x.flatten(1)

    @torch.no_grad()
    def windows(self, mel: torch.Tensor) -> torch.Tensor:
        """A whole clip's mel [frames, 32] -> embeddings of every window at stride 8 [n, 96]."""
        if mel.shape[0] < WINDOW_FRAMES:
            return torch.zeros(0, EMBED_DIM, device=self.device)
        w = mel.unfold(0, WINDOW_FRAMES, STRIDE_FRAMES).transpose(1, 2)
        return self(w)


class WakeHead:
    INPUT = HEAD_FRAMES * EMBED_DIM

    def __init__(self, name: str, weights: dict, device="cpu"):
        self.name, self.device = name, torch.device(device)
        prefix = "model." if any(k.startswith("model.") for k in weights) else ""
        entries: dict[int, dict] = {}
        for k, v in weights.items():
            if k.startswith("verifier_model.") or not k.startswith(prefix):
                continue
            parts = k[len(prefix):].split(".")
            if len(parts) != 2 or not parts[0].isdigit() or parts[1] not in ("weight", "bias"):
                continue
            entries.setdefault(int(parts[0]), {})[parts[1]] = v.float().to(self.device)
        self.layers = []                            # ("linear" | "norm", weight, bias)
        for idx in sorted(entries):
            e = entries[idx]
            if "weight" not in e:
                continue
            self.layers.append(("linear" if e["weight"].dim() == 2 else "norm", e["weight"], e.get("bias")))
        linears = [l for l in self.layers if l[0] == "linear"]
        if not linears or linears[0][1].shape[1] != self.INPUT or linears[-1][1].shape[0] != 1:
            raise ValueError(f"wake head '{name}': expected Linear layers from {self.INPUT} inputs to 1 output")

    @staticmethod
    def from_file(path, name: Optional[str] = None, device="cpu") -> "WakeHead":
        return WakeHead(name or Path(path).stem, load_tensors(path), device)

    @torch.no_grad()
    def __call__(self, features: torch.Tensor) -> torch.Tensor:
        """features [B, 16, 96] (oldest frame first) or [B, 1536] -> probabilities [B]."""
        x = features.to(self.device).float().reshape(-1, self.INPUT)
        last = max(i for i, l in enumerate(self.layers) if l[0] == "linear")
        i = 0
        while i <= last:
            kind, w, b = self.layers[i]
            i += 1
            if kind == "norm":                       # a norm that follows no Linear (not seen in shipped heads)
                x = F.layer_norm(x, (w.numel(),), w, b)
                continue
            x = F.linear(x, w, b)
            if i > last:
                break
            if self.layers[i][0] == "norm":
                x = F.layer_norm(x, (self.layers[i][1].numel(),), *self.layers[i][1:])
                i += 1
            x = F.relu(x)
        return torch.sigmoid(x[:, 0])


class WakeHeadTrainer:
    """1536 -> hidden -> hidden -> 1 with ReLU, trained by Adam on binary cross-entropy."""

    def __init__(self, hidden: int = 128, lr: float = 1e-3, seed: int = 0, device="cpu"):
        torch.manual_seed(seed)
        self.device = torch.device(device)
        self.net = torch.nn.Sequential(torch.nn.Linear(WakeHead.INPUT, hidden), torch.nn.ReLU(), torch.nn.Linear(hidden, hidden),
                                       torch.nn.ReLU(), torch.nn.Linear(hidden, 1)).to(self.device)
        self.opt = torch.optim.Adam(self.net.parameters(), lr=lr)

    def loss(self, batch: torch.Tensor, labels: torch.Tensor, positive_weight: float = 1.0) -> torch.Tensor:
        logits = self.net(batch.to(self.device).float().reshape(-1, WakeHead.INPUT))[:, 0]
        return F.binary_cross_entropy_with_logits(logits, labels.to(self.device).float(),
                                                  pos_weight=torch.tensor(float(positive_weight), device=self.device))

    def step(self, batch: torch.Tensor, labels: torch.Tensor, positive_weight: float = 1.0) -> float:
        self.opt.zero_grad(set_to_none=True)
        loss = self.loss(batch, labels, positive_weight)
        loss.backward()
        self.opt.step()
        return float(loss.detach())

    def fit(self, features: torch.Tensor, labels: torch.Tensor, epochs: int = 30, batch_size: int = 256,
            positive_weight: Optional[float] = None, seed: int = 0) -> list[float]:
        """Mini-batch epochs over [N, 16, 96] windows; returns the mean loss per epoch. The positive weight
        defaults to the negative / positive ratio, since a usable set is mostly negatives."""
        n = features.shape[0]
        pos = float(labels.sum())
        if positive_weight is None:
            positive_weight = max(1.0, (n - pos) / max(pos, 1.0))
        g = torch.Generator().manual_seed(seed)
        history = []
        for _ in range(epochs):
            order = torch.randperm(n, generator=g)
            total = 0.0
            for i in range(0, n, batch_size):
                idx = order[i:i + batch_size]
                total += self.step(features[idx], labels[idx], positive_weight) * idx.numel()
            history.append(total / n)
        return history

    @torch.no_grad()
    def probability(self, features: torch.Tensor) -> torch.Tensor:
        return torch.sigmoid(self.net(features.to(self.device).float().reshape(-1, WakeHead.INPUT))[:, 0])

    def export(self) -> dict:
        """Weights by their ``nn.Sequential`` indices (activations skipped), as :class:`WakeHead` reads them."""
        return {k: v.detach().cpu().contiguous() for k, v in self.net.state_dict().items()}

    def head(self, name: str) -> WakeHead:
        return WakeHead(name, self.export(), self.device)


class SileroVad:
    CHUNK, CONTEXT, HIDDEN = 512, 64, 128

    def __init__(self, weights: Optional[dict] = None, device="cpu", seed: int = 0):
        self.device = torch.device(device)
        if weights is None:
            g = torch.Generator().manual_seed(seed)
            real, imag = dft_basis(256)
            r = lambda *s: torch.randn(*s, generator=g) * (1.0 / math.prod(s[1:])) ** 0.5
            weights = {"stft_conv.weight": torch.cat([real, imag], 0),
                       "conv1.weight": r(128, 129, 3), "conv1.bias": torch.zeros(128), "conv2.weight": r(64, 128, 3), "conv2.bias": torch.zeros(64),
                       "conv3.weight": r(64, 64, 3), "conv3.bias": torch.zeros(64), "conv4.weight": r(128, 64, 3), "conv4.bias": torch.zeros(128),
                       "final_conv.weight": r(1, 128, 1), "final_conv.bias": torch.zeros(1),
                       "lstm_cell.weight_ih": r(512, 128), "lstm_cell.weight_hh": r(512, 128),
                       "lstm_cell.bias_ih": torch.zeros(512), "lstm_cell.bias_hh": torch.zeros(512)}
        self.w = {k: v.float().to(self.device) for k, v in weights.items()}
        self.reset()

    def reset(self, streams: int = 1) -> None:
        self.h = torch.zeros(streams, self.HIDDEN, device=self.device)
        self.c = torch.zeros(streams, self.HIDDEN, device=self.device)
        self.context = torch.zeros(streams, self.CONTEXT, device=self.device)

    @torch.no_grad()
    def __call__(self, chunk: torch.Tensor) -> torch.Tensor:
        """chunk [streams, 512] or [512] at +-1 scale -> speech probability [streams]; state is carried."""
        x = chunk.to(self.device).float()
        if x.dim() == 1:
            x = x[None]
        if x.shape[-1] != self.CHUNK:
            raise ValueError(f"the voice-activity model takes {self.CHUNK} samples per step, got {x.shape[-1]}")
        if x.shape[0] != self.h.shape[0]:
            self.reset(x.shape[0])
        w = self.w
        padded = F.pad(torch.cat([self.context, x], 1)[:, None], (0, 64), mode="reflect")
        self.context = x[:, -self.CONTEXT:].clone()
        spec = F.conv1d(padded, w["stft_conv.weight"], stride=128)
        half = spec.shape[1] // 2
        y = torch.sqrt(spec[:, :half] ** 2 + spec[:, half:] ** 2)
        for name, stride in (("conv1", 1), ("conv2", 2), ("conv3", 2), ("conv4", 1)):
            y = F.relu(F.conv1d(y, w[name + ".weight"], w[name + ".bias"], stride=stride, padding=1))
        gates = F.linear(y[:, :, 0], w["lstm_cell.weight_ih"], w["lstm_cell.bias_ih"]) + \
            F.linear(self.h, w["lstm_cell.weight_hh"], w["lstm_cell.bias_hh"])
        i, f, g, o = gates.chunk(4, 1)
        self.c = torch.sigmoid(f) * self.c + torch.sigmoid(i) * torch.tanh(g)
        self.h = torch.sigmoid(o) * torch.tanh(self.c)
        logit = F.conv1d(F.relu(self.h)[:, :, None], w["final_conv.weight"], w["final_conv.bias"])
        return torch.sigmoid(logit[:, 0, 0])


class VadStream:
    """Turns per-chunk speech probabilities into speech segments: speech starts at ``threshold``, and ends after
    ``min_silence`` seconds below ``threshold - 0.15``. Any number of samples may be pushed."""

    def __init__(self, vad: SileroVad, threshold: float = 0.5, min_silence: float = 0.3):
        self.vad, self.threshold, self.min_silence = vad, threshold, min_silence
        self.reset()

    def reset(self) -> None:
        self.vad.reset()
        self._pending = torch.zeros(0)
        self.consumed, self.speaking, self._start, self._quiet_since = 0, False, 0, None

    def push(self, samples: torch.Tensor) -> list[tuple[str, int]]:
        """-> events ("start" | "end", sample index)."""
        self._pending = torch.cat([self._pending, samples.float().flatten().cpu()])
        events = []
        while self._pending.numel() >= SileroVad.CHUNK:
            chunk, self._pending = self._pending[:SileroVad.CHUNK], self._pending[SileroVad.CHUNK:]
            p = float(self.vad(chunk)[0])
            at = self.consumed
            self.consumed += SileroVad.CHUNK
            if not self.speaking and p >= self.threshold:
                self.speaking, self._quiet_since = True, None
                events.append(("start", at))
            elif self.speaking:
                if p < self.threshold - 0.15:
                    if self._quiet_since is None:
                        self._quiet_since = at
                    if (self.consumed - self._quiet_since) / RATE >= self.min_silence:
                        self.speaking = False
                        events.append(("end", self._quiet_since))
                        self._quiet_since = None
                else:
                    self._quiet_since = None
        return events


@dataclass
class WakeWordSettings:
    threshold: float = 0.5
    smoothing: int = 3                 # score steps (80 ms each) averaged before thresholding
    refractory: float = 2.0            # seconds a word stays quiet after it fired


@dataclass
class WakeDetection:
    word: str
    score: float
    sample_index: int


class WakeDetector:
    """One audio stream. The models are borrowed (stateless, shared between streams); the rings, the smoothing
    history and the refractory clocks live here."""

    def __init__(self, mel: WakeMel, embedding: SpeechEmbedding):
        self.mel, self.embedding = mel, embedding
        self._words: dict[str, list] = {}            # name -> [head, settings, history, quiet-until sample]
        self.reset()

    def add_word(self, head: WakeHead, settings: Optional[WakeWordSettings] = None) -> None:
        self._words[head.name] = [head, settings or WakeWordSettings(), [], 0]

    def remove_word(self, name: str) -> bool:
        return self._words.pop(name, None) is not None

    @property
    def words(self) -> list[str]:
        return list(self._words)

    def reset(self) -> None:
        """After a discontinuity of the stream (a reconnect, a gap): all audio and score state is dropped."""
        self.consumed = 0
        self._pending = torch.zeros(0)
        self._tail = torch.zeros(0)
        self._mel = torch.zeros(0, MEL_BINS)
        self._features = torch.zeros(0, EMBED_DIM)
        for w in self._words.values():
            w[2], w[3] = [], 0

    def push(self, samples: torch.Tensor, feature_sink: Optional[list] = None) -> list[WakeDetection]:
        """Feeds int16-scale samples (any count); returns the words that fired. ``feature_sink`` receives a copy
        of every 16 x 96 window that was scored, so a training set can be built through this very path."""
        self._pending = torch.cat([self._pending, samples.detach().float().flatten().cpu()])
        fired: list[WakeDetection] = []
        while self._pending.numel() >= CHUNK:
            chunk, self._pending = self._pending[:CHUNK], self._pending[CHUNK:]
            self.consumed += CHUNK
            window = torch.cat([self._tail, chunk])
            self._tail = window[-LEFT_CONTEXT:]
            if window.numel() < CHUNK + LEFT_CONTEXT:
                continue                             # the very first chunk has no left context yet
            frames = self.mel(window)[0].cpu()
            self._mel = torch.cat([self._mel, frames])[-(WINDOW_FRAMES + STRIDE_FRAMES):]
            if self._mel.shape[0] < WINDOW_FRAMES:
                continue
            e = self.embedding(self._mel[-WINDOW_FRAMES:][None]).cpu()
            self._features = torch.cat([self._features, e])[-HEAD_FRAMES:]
            if self._features.shape[0] < HEAD_FRAMES:
                continue
            if feature_sink is not None:
                feature_sink.append(self._features.clone())
            for name, w in self._words.items():
                head, settings, history, quiet_until = w
                history.append(float(head(self._features[None])[0]))
                del history[:-max(1, settings.smoothing)]
                score = sum(history) / len(history)
                if score >= settings.threshold and self.consumed >= quiet_until:
                    fired.append(WakeDetection(name, score, self.consumed))
                    w[3] = self.consumed + int(settings.refractory * RATE)
                    history.clear()                 # a fired word must not re-fire on its own tail
        return fired


@torch.no_grad()
def features_for_clips(clips: Iterable[torch.Tensor], mel: WakeMel, embedding: SpeechEmbedding) -> torch.Tensor:
    """Every scored 16 x 96 window of every clip (int16 scale, 16 kHz), through the streaming path: [N, 16, 96]."""
    out: list = []
    det = WakeDetector(mel, embedding)
    for clip in clips:
        det.reset()
        det.push(clip, out)
    return torch.stack(out) if out else torch.zeros(0, HEAD_FRAMES, EMBED_DIM)


def augment(clip: torch.Tensor, copies: int, seed: int = 0, lead: float = 1.6) -> list[torch.Tensor]:
    """Variants of a short clip for training: random gain, background noise, and a random offset inside ``lead``
    seconds of leading room (a head sees 1.28 s ending anywhere in the phrase's tail)."""
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(copies):
        gain = 10 ** (float(torch.empty(1).uniform_(-12, 3, generator=g)) / 20)
        pre = int(float(torch.rand(1, generator=g)) * 0.5 * RATE) + int(lead * RATE)
        post = int(float(torch.rand(1, generator=g)) * 0.3 * RATE) + CHUNK
        x = torch.cat([torch.zeros(pre), clip.float() * gain, torch.zeros(post)])
        level = 10 ** (float(torch.empty(1).uniform_(-45, -25, generator=g)) / 20) * 32768.0
        out.append(x + torch.randn(x.numel(), generator=g) * level)
    return out


def train_wake_word(models: "WakeModelSet", name: str, positives: list, negatives: list, epochs: int = 40, hidden: int = 128,
                    copies: int = 8, tail_windows: int = 3, seed: int = 0, log: Optional[Callable[[str], None]] = None) -> dict:
    """Trains and stores the head for ``name``. ``positives``: clips (int16 scale, 16 kHz) that END with the phrase;
    only the last ``tail_windows`` scored windows of each augmented copy count as positive (the ones that have heard
    the whole phrase), the earlier ones of those copies are dropped. ``negatives``: any other audio, every window."""
    pos_feats = []
    for i, clip in enumerate(positives):
        for v in augment(clip, copies, seed + 97 * i):
            f = features_for_clips([v], models.mel, models.embedding)
            if f.shape[0]:
                pos_feats.append(f[-tail_windows:])
    neg = features_for_clips(negatives, models.mel, models.embedding)
    if not pos_feats or neg.shape[0] == 0:
        raise ValueError("training needs at least one usable positive clip and some negative audio (each over 2.1 s)")
    pos = torch.cat(pos_feats)
    x = torch.cat([pos, neg])
    y = torch.cat([torch.ones(len(pos)), torch.zeros(len(neg))])
    trainer = WakeHeadTrainer(hidden, seed=seed, device=models.device)
    history = trainer.fit(x, y, epochs=epochs, seed=seed)
    p = trainer.probability(x).cpu()
    report = {"positives": len(pos), "negatives": len(neg), "loss": history[-1],
              "recall": float((p[:len(pos)] >= 0.5).float().mean()), "false_accepts": float((p[len(pos):] >= 0.5).float().mean())}
    if log:
        log(f"{name}: {report}")
    report["path"] = str(models.save_head(name, trainer.export()))
    return report


class WakeModelSet:
    """The shared models of a deployment, from one directory: ``melspectrogram.onnx``, ``embedding_model.onnx``,
    optional ``silero_vad_16k.safetensors``, and one head file per wake word (``<word>.onnx`` / ``.safetensors``)."""

    SHARED = {"melspectrogram", "embedding_model", "silero_vad", "silero_vad_16k"}

    def __init__(self, directory, device="cpu"):
        d = Path(directory)
        self.directory, self.device = d, device
        find = lambda stem: next((d / f"{stem}{ext}" for ext in (".onnx", ".safetensors") if (d / f"{stem}{ext}").exists()), None)
        mel_file, emb_file = find("melspectrogram"), find("embedding_model")
        if mel_file is None or emb_file is None:
            raise FileNotFoundError(f"{d}: melspectrogram / embedding_model (.onnx or .safetensors) are required")
        self.mel = WakeMel(load_tensors(mel_file), device)
        self.embedding = SpeechEmbedding(load_tensors(emb_file), device)
        vad_file = find("silero_vad_16k") or find("silero_vad")
        self.vad_weights = load_tensors(vad_file) if vad_file is not None else None
        self.heads = {}
        for f in sorted(d.iterdir()):
            if f.suffix in (".onnx", ".safetensors") and f.stem not in self.SHARED:
                try:
                    self.heads[f.stem] = WakeHead.from_file(f, device=device)
                except ValueError:
                    continue                        # not a wake head

    def detector(self, settings: Optional[dict] = None) -> WakeDetector:
        det = WakeDetector(self.mel, self.embedding)
        for name, head in self.heads.items():
            det.add_word(head, (settings or {}).get(name))
        return det

    def vad(self) -> Optional[SileroVad]:
        return SileroVad(self.vad_weights, self.device) if self.vad_weights is not None else None

    def save_head(self, name: str, tensors: dict) -> Path:
        from ..assets.safetensors import save_file
        path = self.directory / f"{name}.safetensors"
        save_file(tensors, path)
        self.heads[name] = WakeHead(name, tensors, self.device)
        return path
