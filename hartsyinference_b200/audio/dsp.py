"""STFT, mel filterbank and log-mel features (the Whisper front end and the generic pieces the
vocoder / TTS models share).

Reference: Backends/IBackend.cs (`Fft`, `Stft`, `MelFilterbank` ops),
src/HartsyInference.Audio/Frontends/, src/HartsyInference.Audio/Preprocessing/.
"""
from __future__ import annotations

import math

import torch


def hann_window(n: int, periodic: bool = True) -> torch.Tensor:
    return torch.hann_window(n, periodic=periodic, dtype=torch.float32)


def _hz_to_mel_slaney(f: torch.Tensor) -> torch.Tensor:
    f_sp, min_log_hz = 200.0 / 3, 1000.0
    min_log_mel, logstep = min_log_hz / f_sp, math.log(6.4) / 27.0
    return torch.where(f >= min_log_hz, min_log_mel + torch.log(f.clamp_min(1e-10) / min_log_hz) / logstep, f / f_sp)


def _mel_to_hz_slaney(m: torch.Tensor) -> torch.Tensor:
    f_sp, min_log_hz = 200.0 / 3, 1000.0
    min_log_mel, logstep = min_log_hz / f_sp, math.log(6.4) / 27.0
    return torch.where(m >= min_log_mel, min_log_hz * torch.exp(logstep * (m - min_log_mel)), m * f_sp)


def mel_filterbank(n_mels: int, n_fft: int, rate: int, f_min: float = 0.0, f_max: float | None = None,
                   htk: bool = False, norm_slaney: bool = True) -> torch.Tensor:
    """Triangular filters [n_mels, n_fft // 2 + 1]; Slaney scale with area normalisation by default
    (what librosa and Whisper use), HTK scale optionally."""
    f_max = f_max if f_max is not None else rate / 2
    freqs = torch.linspace(0, rate / 2, n_fft // 2 + 1, dtype=torch.float64)
    lo, hi = torch.tensor(f_min, dtype=torch.float64), torch.tensor(f_max, dtype=torch.float64)
    if htk:
        to_mel = lambda f: 2595.0 * torch.log10(1.0 + f / 700.0)      # noqa: E731
        to_hz = lambda m: 700.0 * (10.0 ** (m / 2595.0) - 1.0)        # noqa: E731
    else:
        to_mel, to_hz = _hz_to_mel_slaney, _mel_to_hz_slaney
    pts = to_hz(torch.linspace(float(to_mel(lo)), float(to_mel(hi)), n_mels + 2, dtype=torch.float64))
    diff = pts[1:] - pts[:-1]
    ramps = pts[:, None] - freqs[None]
    lower = -ramps[:-2] / diff[:-1, None]
    upper = ramps[2:] / diff[1:, None]
    fb = torch.minimum(lower, upper).clamp_min(0)
    if norm_slaney:
        fb = fb * (2.0 / (pts[2:] - pts[:-2]))[:, None]
    return fb.to(torch.float32)


def stft_power(x: torch.Tensor, n_fft: int, hop: int, window: torch.Tensor | None = None, center: bool = True) -> torch.Tensor:
    """|STFT|^2 of x [n] -> [n_fft // 2 + 1, frames] (reflect padding when ``center``)."""
    window = (window if window is not None else hann_window(n_fft)).to(x.device)
    spec = torch.stft(x.float(), n_fft, hop, window=window, center=center, pad_mode="reflect", return_complex=True)
    return spec.abs() ** 2


def log_mel_spectrogram(audio: torch.Tensor, n_mels: int = 80, rate: int = 16000, n_fft: int = 400, hop: int = 160,
                        chunk_seconds: float | None = 30.0) -> torch.Tensor:
    """Whisper's input features: pad / trim to ``chunk_seconds``, power STFT without its last frame,
    mel, log10 clamped to 8 dB below the maximum, (x + 4) / 4. -> [n_mels, frames]."""
    x = audio.float().flatten()
    if chunk_seconds is not None:
        n = int(chunk_seconds * rate)
        x = torch.nn.functional.pad(x, (0, max(0, n - x.numel())))[:n]
    power = stft_power(x, n_fft, hop)[:, :-1]
    mel = mel_filterbank(n_mels, n_fft, rate).to(power.device) @ power
    lg = torch.log10(mel.clamp_min(1e-10))
    lg = torch.maximum(lg, lg.max() - 8.0)
    return (lg + 4.0) / 4.0
