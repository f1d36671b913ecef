"""Frame tensors -> video files.

``encode_video`` pipes raw RGB frames into ``ffmpeg`` (H.264 / yuv420p by default) when the
binary is on PATH; otherwise, or on request, frames are written as a numbered PNG or BMP sequence
plus a small JSON manifest (fps, size, frame count) so that the clip can be muxed elsewhere.

Reference: src/HartsyInference.Video/Encoding/ (ffmpeg subprocess encoder / muxer, BMP sequence
fallback).
"""
from __future__ import annotations

import json
import shutil
import subprocess
from pathlib import Path
from typing import Optional

import torch

from ..utils import png


def ffmpeg_path() -> Optional[str]:
    return shutil.which("ffmpeg")


def frames_to_uint8(frames: torch.Tensor) -> torch.Tensor:
    """[F, 3, H, W] or [3, F, H, W] or [F, H, W, 3] in [-1, 1] / [0, 1] / uint8 -> uint8 [F, H, W, 3]."""
    f = frames.detach().cpu()
    if f.dim() != 4:
        raise ValueError("expected a 4-D frame tensor")
    if f.shape[-1] != 3:
        if f.shape[1] == 3:
            f = f.permute(0, 2, 3, 1)
        elif f.shape[0] == 3:
            f = f.permute(1, 2, 3, 0)
        else:
            raise ValueError(f"cannot find the colour axis in {tuple(frames.shape)}")
    if f.dtype != torch.uint8:
        f = f.float()
        if f.min() < 0:
            f = (f + 1) / 2
        f = (f.clamp(0, 1) * 255 + 0.5).to(torch.uint8)
    return f.contiguous()


class FrameSequenceWriter:
    """Numbered image files + manifest.json in a directory."""

    def __init__(self, directory, fmt: str = "png", fps: float = 16.0):
        if fmt not in ("png", "bmp"):
            raise ValueError("fmt must be png or bmp")
        self.dir = Path(directory)
        self.dir.mkdir(parents=True, exist_ok=True)
        self.fmt, self.fps, self.count, self.size = fmt, fps, 0, None

    def add(self, frame_u8: torch.Tensor) -> Path:
        h, w, _ = frame_u8.shape
        self.size = (w, h)
        p = self.dir / f"frame_{self.count:06d}.{self.fmt}"
        rgb = frame_u8.contiguous().numpy().tobytes()
        if self.fmt == "png":
            p.write_bytes(png.encode_png(rgb, w, h))
        else:
            png.write_bmp(str(p), rgb, w, h)
        self.count += 1
        return p

    def close(self) -> Path:
        m = self.dir / "manifest.json"
        m.write_text(json.dumps({"fps": self.fps, "frames": self.count, "width": self.size[0] if self.size else 0,
                                 "height": self.size[1] if self.size else 0, "pattern": f"frame_%06d.{self.fmt}"}))
        return m


def encode_video(frames: torch.Tensor, path, fps: float = 16.0, codec: str = "libx264", crf: int = 18,
                 allow_fallback: bool = True) -> Path:
    """Writes ``path`` (e.g. out.mp4). Returns the file written, or the sequence directory
    (``path`` without its suffix) when ffmpeg is missing and the fallback is allowed."""
    f = frames_to_uint8(frames)
    n, h, w, _ = f.shape
    path = Path(path)
    exe = ffmpeg_path()
    if exe is None:
        if not allow_fallback:
            raise RuntimeError("ffmpeg is not installed")
        seq = FrameSequenceWriter(path.with_suffix(""), "png", fps)
        for i in range(n):
            seq.add(f[i])
        seq.close()
        return seq.dir
    cmd = [exe, "-y", "-loglevel", "error", "-f", "rawvideo", "-pix_fmt", "rgb24", "-s", f"{w}x{h}", "-r", str(fps),
           "-i", "-", "-an", "-c:v", codec, "-pix_fmt", "yuv420p", "-crf", str(crf), str(path)]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stderr=subprocess.PIPE)
    try:
        proc.stdin.write(f.numpy().tobytes())
        proc.stdin.close()
    except BrokenPipeError:
        pass
    err = proc.stderr.read().decode(errors="replace")
    if proc.wait() != 0:
        raise RuntimeError(f"ffmpeg failed: {err.strip()[:400]}")
    return path
