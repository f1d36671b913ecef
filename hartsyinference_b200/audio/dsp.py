"""STFT, mel filterbank and log-mel features (the Whisper front end and the generic pieces the
vocoder / TTS models share).

Reference: Backends/IBackend.cs (`Fft`, `Stft`, `MelFilterbank` ops),
src/HartsyInference.Audio/Frontends/, src/HartsyInference.Audio/Preprocessing/.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


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


# ---------------------------------------------------------------------------------------- output level
SILENCE_PEAK = 1e-4


def normalize_peak(audio: torch.Tensor, peak: float = 0.95) -> torch.Tensor:
    """Scales ``audio`` so that its largest absolute sample equals ``peak``; silence is returned as it is.
    (A product step after synthesis, not part of any model: parity checks run without it.
    Reference: src/HartsyInference.Audio/Preprocessing/LoudnessNormalizer.cs.)"""
    top = float(audio.abs().max()) if audio.numel() else 0.0
    return audio if top < SILENCE_PEAK else audio * (peak / top)


def normalize_rms(audio: torch.Tensor, target_rms: float = 0.1, peak_ceiling: float = 0.95) -> torch.Tensor:
    """Scales to a target RMS (even loudness across clips); the gain is capped so the peak stays under the ceiling."""
    top = float(audio.abs().max()) if audio.numel() else 0.0
    if top < SILENCE_PEAK:
        return audio
    rms = float(audio.float().pow(2).mean().sqrt())
    return audio * min(target_rms / max(rms, 1e-12), peak_ceiling / top)


# ---------------------------------------------------------------------------------------- pitch
def estimate_f0(audio: torch.Tensor, rate: int = 16000, hop: int = 320, f_min: float = 50.0, f_max: float = 1100.0,
                threshold: float = 0.15) -> torch.Tensor:
    """YIN pitch contour: one value per hop in Hz, 0 where unvoiced. All frames are processed at once:
    difference function through FFT autocorrelation, cumulative-mean normalisation, the first dip under
    ``threshold`` (its local minimum), parabolic refinement. At 16 kHz with hop 320 the contour lines up with
    HuBERT frames. Reference: src/HartsyInference.Audio/Dsp/F0Estimator.cs."""
    x = audio.float().flatten()
    tau_max = int(rate / f_min)
    tau_min = max(2, int(rate / f_max))
    win = 2 * tau_max
    n = x.numel() // hop
    if n == 0:
        return torch.zeros(0)
    pad = F.pad(x, (0, win + tau_max))
    frames = pad.unfold(0, win + tau_max, hop)[:n]                                  # [n, win + tau_max]
    # d(tau) = sum_j (x_j - x_{j+tau})^2 over j < win  =  e(0) + e(tau) - 2 r(tau)
    size = 1 << (win + tau_max).bit_length()
    head = frames[:, :win]
    spec = torch.fft.rfft(frames, size) * torch.fft.rfft(head, size).conj()
    corr = torch.fft.irfft(spec, size)[:, :tau_max + 1]                              # r(tau) = sum_j head_j frame_{j+tau}
    sq = F.pad(frames.pow(2).cumsum(1), (1, 0))
    energy = sq[:, win:win + tau_max + 1] - sq[:, :tau_max + 1]                      # e(tau) = sum_j frame_{j+tau}^2
    diff = (energy[:, :1] + energy - 2 * corr).clamp_min(0)
    cm = diff[:, 1:] * torch.arange(1, tau_max + 1) / diff[:, 1:].cumsum(1).clamp_min(1e-12)
    cmnd = torch.cat([torch.ones(n, 1), cm], 1)                                      # [n, tau_max + 1]
    search = cmnd[:, tau_min:]
    below = search < threshold
    first = torch.where(below.any(1), below.float().argmax(1), torch.full((n,), -1))
    out = torch.zeros(n)
    for i in range(n):                                   # walk down to the local minimum of the first dip
        t = int(first[i])
        if t < 0:
            continue
        t += tau_min
        while t + 1 <= tau_max and cmnd[i, t + 1] < cmnd[i, t]:
            t += 1
        if 1 <= t < tau_max:
            a, b, c = float(cmnd[i, t - 1]), float(cmnd[i, t]), float(cmnd[i, t + 1])
            den = a - 2 * b + c
            shift = 0.5 * (a - c) / den if abs(den) > 1e-12 else 0.0
        else:
            shift = 0.0
        out[i] = rate / (t + shift)
    return out


# ---------------------------------------------------------------------------------------- Kaldi filter bank
def kaldi_fbank(audio: torch.Tensor, rate: int = 16000, n_mels: int = 80, frame_ms: float = 25.0, shift_ms: float = 10.0,
                low_freq: float = 20.0, high_freq: float = 0.0, preemphasis: float = 0.97) -> torch.Tensor:
    """Kaldi-style log mel filter-bank features [frames, n_mels] (what CAM++-class speaker encoders take): frames
    without padding (a trailing partial frame is dropped), per-frame mean removal, pre-emphasis with the first
    sample repeated, Povey window (Hann^0.85), power spectrum at the next power of two, triangular filters evenly
    spaced on the ``1127 ln(1 + f / 700)`` scale between ``low_freq`` and Nyquist (+ ``high_freq`` when <= 0),
    natural log with a floor at machine epsilon, no dither. Samples are taken as given (Kaldi tools scale to
    int16 first). Reference: src/HartsyInference.Audio/Preprocessing/KaldiFbankExtractor.cs."""
    x = audio.float().flatten()
    flen, shift = int(rate * frame_ms / 1000), int(rate * shift_ms / 1000)
    if x.numel() < flen:
        return torch.zeros(0, n_mels)
    frames = x.unfold(0, flen, shift)
    frames = frames - frames.mean(1, keepdim=True)
    frames = torch.cat([frames[:, :1] * (1 - preemphasis), frames[:, 1:] - preemphasis * frames[:, :-1]], 1)
    window = (0.5 - 0.5 * torch.cos(2 * math.pi * torch.arange(flen) / (flen - 1))).pow(0.85)
    nfft = 1 << (flen - 1).bit_length()
    power = torch.fft.rfft(frames * window, nfft).abs().pow(2)                        # [frames, nfft / 2 + 1]
    nyquist = rate / 2
    high = nyquist + high_freq if high_freq <= 0 else high_freq
    mel = lambda f: 1127.0 * math.log(1.0 + f / 700.0)
    lo_m, hi_m = mel(low_freq), mel(high)
    delta = (hi_m - lo_m) / (n_mels + 1)
    bins = 1127.0 * torch.log(1.0 + torch.arange(nfft // 2) * (rate / nfft) / 700.0)   # Kaldi leaves the Nyquist bin out
    left = lo_m + torch.arange(n_mels)[:, None] * delta
    centre, right = left + delta, left + 2 * delta
    up, down = (bins[None] - left) / (centre - left), (right - bins[None]) / (right - centre)
    bank = torch.minimum(up, down).clamp_min(0)                                       # [n_mels, nfft / 2]
    feats = power[:, :nfft // 2] @ bank.t()
    return torch.log(feats.clamp_min(torch.finfo(torch.float32).eps))
