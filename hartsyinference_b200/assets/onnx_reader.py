"""Weights out of an ONNX file without the onnx package: a protobuf wire-format walk over
``ModelProto.graph.initializer`` that returns every initialiser as a tensor. Only what a weight
reader needs is decoded (names, dims, data type, raw / typed data); nodes are skipped.

Reference: src/HartsyInference.ModelAssets/ (ONNX initialiser reader used by the Piper / Kokoro /
detector checkpoints).
"""
from __future__ import annotations

from pathlib import Path
from typing import Iterator

import numpy as np
import torch

# TensorProto.DataType -> numpy dtype
_DT = {1: np.float32, 2: np.uint8, 3: np.int8, 4: np.uint16, 5: np.int16, 6: np.int32, 7: np.int64, 9: np.bool_,
       10: np.float16, 11: np.float64, 12: np.uint32, 13: np.uint64}
_BF16 = 16


def _varint(buf: bytes, pos: int) -> tuple[int, int]:
    out, shift = 0, 0
    while True:
        b = buf[pos]
        pos += 1
        out |= (b & 0x7F) << shift
        if b < 0x80:
            return out, pos
        shift += 7
        if shift > 70:
            raise ValueError("malformed varint")


def _fields(buf: bytes, start: int = 0, end: int | None = None) -> Iterator[tuple[int, int, object]]:
    """(field number, wire type, value) for one message; length-delimited values are (start, end) spans."""
    pos, end = start, len(buf) if end is None else end
    if end > len(buf):
        raise ValueError("protobuf field runs past the end of the file")
    while pos < end:
        key, pos = _varint(buf, pos)
        num, wt = key >> 3, key & 7
        if wt == 0:
            v, pos = _varint(buf, pos)
            yield num, wt, v
        elif wt == 1:
            yield num, wt, buf[pos:pos + 8]
            pos += 8
        elif wt == 2:
            n, pos = _varint(buf, pos)
            yield num, wt, (pos, pos + n)
            pos += n
        elif wt == 5:
            yield num, wt, buf[pos:pos + 4]
            pos += 4
        else:
            raise ValueError(f"unsupported protobuf wire type {wt}")
    if pos != end:
        raise ValueError("truncated protobuf message")


def _signed(v: int) -> int:
    return v - (1 << 64) if v >= (1 << 63) else v


def _packed_varints(buf: bytes, span) -> list[int]:
    pos, end = span
    out = []
    while pos < end:
        v, pos = _varint(buf, pos)
        out.append(_signed(v))
    return out


def _tensor(buf: bytes, span, base_dir: Path | None) -> tuple[str, torch.Tensor]:
    dims: list[int] = []
    dtype, name, raw = 1, "", None
    floats: list = []
    ints: list[int] = []
    doubles: list = []
    external: dict[str, str] = {}
    location = 0
    for num, wt, v in _fields(buf, *span):
        if num == 1:
            dims += _packed_varints(buf, v) if wt == 2 else [_signed(v)]
        elif num == 2:
            dtype = v
        elif num == 4:
            floats.append(np.frombuffer(buf[v[0]:v[1]], "<f4") if wt == 2 else np.frombuffer(v, "<f4"))
        elif num in (5, 7):
            ints += _packed_varints(buf, v) if wt == 2 else [_signed(v)]
        elif num == 8:
            name = buf[v[0]:v[1]].decode("utf-8")
        elif num == 9:
            raw = buf[v[0]:v[1]]
        elif num == 10:
            doubles.append(np.frombuffer(buf[v[0]:v[1]], "<f8") if wt == 2 else np.frombuffer(v, "<f8"))
        elif num == 13:            # external_data: repeated StringStringEntryProto {key=1, value=2}
            kv = {n: buf[s[0]:s[1]].decode("utf-8") for n, w, s in _fields(buf, *v) if w == 2}
            external[kv.get(1, "")] = kv.get(2, "")
        elif num == 14:
            location = v
    if location == 1 and external:
        if base_dir is None:
            raise ValueError(f"initialiser '{name}' keeps its data in an external file")
        with open(base_dir / external["location"], "rb") as f:
            f.seek(int(external.get("offset", "0")))
            raw = f.read(int(external["length"])) if "length" in external else f.read()
    if dtype == _BF16:
        arr = np.frombuffer(raw, "<u2") if raw is not None else np.asarray(ints, "<u2")
        t = torch.from_numpy(arr.astype(np.int16).copy()).view(torch.bfloat16)
    else:
        if dtype not in _DT:
            raise ValueError(f"initialiser '{name}': unsupported ONNX data type {dtype}")
        np_dt = np.dtype(_DT[dtype])
        if raw is not None:
            arr = np.frombuffer(raw, np_dt.newbyteorder("<"))
        elif floats:
            arr = np.concatenate(floats).astype(np_dt)
        elif doubles:
            arr = np.concatenate(doubles).astype(np_dt)
        elif dtype == 10:          # float16 values travel as their bit patterns in int32_data
            arr = np.asarray(ints, np.uint16).view(np.float16)
        else:
            arr = np.asarray(ints).astype(np_dt)
        t = torch.from_numpy(arr.astype(np_dt, copy=True))
    return name, t.reshape([int(d) for d in dims])


def read_onnx_initializers(path) -> dict[str, torch.Tensor]:
    """{initialiser name: tensor} of the model at ``path`` (external data files are read from its folder)."""
    p = Path(path)
    buf = p.read_bytes()
    out: dict[str, torch.Tensor] = {}
    for num, wt, v in _fields(buf):
        if num == 7 and wt == 2:                      # ModelProto.graph
            for gnum, gwt, gv in _fields(buf, *v):
                if gnum == 5 and gwt == 2:            # GraphProto.initializer
                    name, t = _tensor(buf, gv, p.parent)
                    out[name] = t
    return out
