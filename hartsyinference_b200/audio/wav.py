"""RIFF/WAVE reading and writing (PCM 8/16/24/32-bit, IEEE float 32/64) and band-limited resampling.

Reference: src/HartsyInference.Audio/Io/WavFile.cs, src/HartsyInference.Audio/Io/Resampler.cs.
"""
from __future__ import annotations

import math
import struct
from pathlib import Path
from typing import Union

import numpy as np
import torch


def read_wav(src: Union[str, Path, bytes]) -> tuple[torch.Tensor, int]:
    """-> (samples float32 [channels, n] in [-1, 1], sample rate). Walks the chunk list, so extra
    chunks (LIST, fact, ...) before ``data`` are skipped; WAVE_FORMAT_EXTENSIBLE is resolved through
    its sub-format."""
    raw = src if isinstance(src, (bytes, bytearray)) else Path(src).read_bytes()
    if len(raw) < 12 or raw[:4] != b"RIFF" or raw[8:12] != b"WAVE":
        raise ValueError("not a RIFF/WAVE file")
    pos, fmt, data = 12, None, None
    while pos + 8 <= len(raw):
        cid, size = raw[pos:pos + 4], struct.unpack_from("<I", raw, pos + 4)[0]
        body = raw[pos + 8: pos + 8 + size]
        if cid == b"fmt ":
            tag, ch, rate, _, _, bits = struct.unpack_from("<HHIIHH", body, 0)
            if tag == 0xFFFE and len(body) >= 26:
                tag = struct.unpack_from("<H", body, 24)[0]
            fmt = (tag, ch, rate, bits)
        elif cid == b"data":
            data = body
        pos += 8 + size + (size & 1)
    if fmt is None or data is None:
        raise ValueError("WAV file without fmt or data chunk")
    tag, ch, rate, bits = fmt
    if tag == 1:
        if bits == 8:
            x = (np.frombuffer(data, np.uint8).astype(np.float32) - 128.0) / 128.0
        elif bits == 16:
            x = np.frombuffer(data, "<i2").astype(np.float32) / 32768.0
        elif bits == 24:
            b = np.frombuffer(data[: len(data) // 3 * 3], np.uint8).reshape(-1, 3).astype(np.int32)
            v = b[:, 0] | (b[:, 1] << 8) | (b[:, 2] << 16)
            x = np.where(v & 0x800000, v - (1 << 24), v).astype(np.float32) / 8388608.0
        elif bits == 32:
            x = np.frombuffer(data, "<i4").astype(np.float32) / 2147483648.0
        else:
            raise ValueError(f"unsupported PCM width {bits}")
    elif tag == 3:
        x = np.frombuffer(data, "<f4" if bits == 32 else "<f8").astype(np.float32)
    else:
        raise ValueError(f"unsupported WAV format tag {tag}")
    n = len(x) // ch
    return torch.from_numpy(x[: n * ch].reshape(n, ch).T.copy()), rate


def write_wav(dst: Union[str, Path, None], samples: torch.Tensor, rate: int, float32: bool = False) -> bytes:
    """samples [n] or [channels, n] in [-1, 1] -> 16-bit PCM (or float32) WAV bytes, also written to
    ``dst`` when it is a path."""
    x = samples.detach().float().cpu()
    if x.ndim == 1:
        x = x[None]
    ch, n = x.shape
    inter = x.T.contiguous().numpy()
    if float32:
        body, tag, bits = inter.astype("<f4").tobytes(), 3, 32
    else:
        body, tag, bits = (np.clip(inter, -1.0, 1.0) * 32767.0).round().astype("<i2").tobytes(), 1, 16
    hdr = struct.pack("<4sI4s4sIHHIIHH4sI", b"RIFF", 36 + len(body), b"WAVE", b"fmt ", 16, tag, ch, rate,
                      rate * ch * bits // 8, ch * bits // 8, bits, b"data", len(body))
    out = hdr + body
    if dst is not None:
        Path(dst).write_bytes(out)
    return out


def resample(x: torch.Tensor, src_rate: int, dst_rate: int, taps: int = 16) -> torch.Tensor:
    """Windowed-sinc polyphase resampling along the last dim (Hann window, ``taps`` zero crossings
    each side, cut-off at the lower Nyquist)."""
    if src_rate == dst_rate:
        return x
    g = math.gcd(src_rate, dst_rate)
    up, down = dst_rate // g, src_rate // g
    cutoff = 0.5 * min(1.0, up / down) * 2.0          # relative to the source Nyquist
    width = math.ceil(taps / cutoff)
    idx = torch.arange(-width, width + down, dtype=torch.float64)
    phases = []
    for p in range(up):
        t = (idx - p * down / up) * cutoff               # fractional delay of output phase p
        w = torch.where(t.abs() < taps, torch.cos(t * math.pi / taps / 2) ** 2, torch.zeros_like(t))
        k = torch.sinc(t) * w * cutoff
        phases.append(k)
    kern = torch.stack(phases).to(torch.float32)[:, None]           # [up, 1, K]
    shape = x.shape
    y = x.reshape(-1, 1, shape[-1]).float()
    y = torch.nn.functional.pad(y, (width, width + down))
    y = torch.nn.functional.conv1d(y, kern.to(y.device), stride=down)   # [B, up, frames]
    y = y.transpose(1, 2).reshape(y.shape[0], -1)
    n_out = math.ceil(shape[-1] * up / down)
    return y[:, :n_out].reshape(*shape[:-1], n_out)
