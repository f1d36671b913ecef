"""Minimal PNG encoder (RGB24, zlib) and BMP writer, so that image results can leave the process
without an imaging library (the reference ships its own PngEncoder, src/HartsyInference.Engine/
PngEncoder.cs, and a BMP-sequence fallback for video, src/HartsyInference.Video/Encoding/)."""
from __future__ import annotations

import struct
import zlib


def _chunk(tag: bytes, data: bytes) -> bytes:
    return struct.pack(">I", len(data)) + tag + data + struct.pack(">I", zlib.crc32(tag + data) & 0xFFFFFFFF)


def encode_png(rgb: bytes, width: int, height: int, level: int = 3) -> bytes:
    assert len(rgb) == width * height * 3
    stride = width * 3
    raw = b"".join(b"\x00" + rgb[y * stride:(y + 1) * stride] for y in range(height))
    return (b"\x89PNG\r\n\x1a\n" + _chunk(b"IHDR", struct.pack(">IIBBBBB", width, height, 8, 2, 0, 0, 0)) +
            _chunk(b"IDAT", zlib.compress(raw, level)) + _chunk(b"IEND", b""))


def write_bmp(path: str, rgb: bytes, width: int, height: int) -> None:
    row = (width * 3 + 3) & ~3
    pad = b"\0" * (row - width * 3)
    body = bytearray()
    for y in range(height - 1, -1, -1):
        line = rgb[y * width * 3:(y + 1) * width * 3]
        body += bytes(b for i in range(0, len(line), 3) for b in (line[i + 2], line[i + 1], line[i])) + pad
    with open(path, "wb") as f:
        f.write(b"BM" + struct.pack("<IHHI", 54 + len(body), 0, 0, 54))
        f.write(struct.pack("<IiiHHIIiiII", 40, width, height, 1, 24, 0, len(body), 2835, 2835, 0, 0))
        f.write(body)
