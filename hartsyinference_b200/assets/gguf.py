"""GGUF reader / writer and block codecs (C++ core in ``csrc/runtime/gguf.cpp``).

``GgufFile`` exposes the key/value metadata as a dict and tensors either raw (packed blocks, for
the device dequant-GEMM path) or dequantised to fp32. ``write_gguf`` produces v3 files, with
optional quantisation to Q8_0 / Q4_0 / Q4_K. Counterparts: GgufLoader, GgufModelLoader, GgufWriter,
GgufQuantizer (src/HartsyInference.ModelAssets/Gguf/).
"""
from __future__ import annotations

import ctypes as C
import json
import struct
from pathlib import Path
from typing import Optional

import numpy as np
import torch

from .. import runtime
from ..exceptions import HartsyInferenceError

GGML_TYPES = {"F32": 0, "F16": 1, "Q4_0": 2, "Q4_1": 3, "Q5_0": 6, "Q5_1": 7, "Q8_0": 8, "Q2_K": 10, "Q3_K": 11,
              "Q4_K": 12, "Q5_K": 13, "Q6_K": 14, "IQ4_NL": 20, "BF16": 30, "MXFP4": 39}
MXFP4 = 39            # 32 elements: one E8M0 scale byte + 16 bytes of E2M1 nibbles (element j low, j + 16 high)
GGML_NAMES = {v: k for k, v in GGML_TYPES.items()}

_bound = False


def _lib():
    global _bound
    L = runtime.lib()
    if not _bound:
        vp, i32, i64, u64, cs = C.c_void_p, C.c_int32, C.c_int64, C.c_uint64, C.c_char_p
        for name, res, args in (
            ("b200_gguf_open", vp, [cs]), ("b200_gguf_error", cs, [vp]), ("b200_gguf_close", None, [vp]),
            ("b200_gguf_metadata", cs, [vp]), ("b200_gguf_version", i32, [vp]), ("b200_gguf_count", i32, [vp]),
            ("b200_gguf_name", cs, [vp, i32]), ("b200_gguf_type", i32, [vp, i32]), ("b200_gguf_ndim", i32, [vp, i32]),
            ("b200_gguf_dims", None, [vp, i32, C.POINTER(i64)]), ("b200_gguf_data", vp, [vp, i32, C.POINTER(u64)]),
            ("b200_ggml_type_info", i32, [i32, C.POINTER(i32), C.POINTER(i32), cs, i32]),
            ("b200_ggml_dequant", i32, [i32, vp, vp, i64]), ("b200_ggml_quant", i32, [i32, vp, vp, i64]),
        ):
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _bound = True
    return L


def type_geometry(ggml_type: int) -> tuple[int, int]:
    """(elements per block, bytes per block)."""
    b, n = C.c_int32(), C.c_int32()
    if _lib().b200_ggml_type_info(ggml_type, C.byref(b), C.byref(n), None, 0) != 0:
        raise HartsyInferenceError(f"unknown ggml type {ggml_type}")
    return b.value, n.value


def dequantize(raw: torch.Tensor | np.ndarray | bytes, ggml_type: int, numel: int) -> torch.Tensor:
    """Packed blocks -> fp32 [numel]."""
    if isinstance(raw, torch.Tensor):
        raw = raw.contiguous().view(torch.uint8).numpy()
    buf = np.frombuffer(raw, dtype=np.uint8) if isinstance(raw, (bytes, bytearray)) else np.ascontiguousarray(raw)
    out = np.empty(numel, dtype=np.float32)
    rc = _lib().b200_ggml_dequant(ggml_type, buf.ctypes.data, out.ctypes.data, numel)
    if rc != 0:
        raise HartsyInferenceError(f"cannot dequantise ggml type {GGML_NAMES.get(ggml_type, ggml_type)} (code {rc})")
    return torch.from_numpy(out)


def quantize(x: torch.Tensor, ggml_type: int) -> torch.Tensor:
    """fp32 tensor -> packed blocks (uint8 [nbytes]); supports Q8_0, Q4_0, Q4_K, MXFP4."""
    if ggml_type == MXFP4:
        from .lowbit import E2M1_MAX, e2m1_encode, e8m0_decode, e8m0_from_amax
        xb = x.detach().float().cpu().reshape(-1, 32)
        sc = e8m0_from_amax(xb.abs().amax(-1), E2M1_MAX)
        codes = e2m1_encode(xb / e8m0_decode(sc)[:, None])
        packed = (codes[:, :16] | (codes[:, 16:] << 4)).to(torch.uint8)
        return torch.cat([sc[:, None], packed], 1).reshape(-1)
    blk, nb = type_geometry(ggml_type)
    xf = np.ascontiguousarray(x.detach().float().cpu().numpy().reshape(-1))
    if xf.size % blk:
        raise HartsyInferenceError(f"{xf.size} elements are not a multiple of the {blk}-element block")
    out = np.empty(xf.size // blk * nb, dtype=np.uint8)
    rc = _lib().b200_ggml_quant(ggml_type, xf.ctypes.data, out.ctypes.data, xf.size)
    if rc != 0:
        raise HartsyInferenceError(f"cannot quantise to ggml type {GGML_NAMES.get(ggml_type, ggml_type)} (code {rc})")
    return torch.from_numpy(out)


class GgufFile:
    def __init__(self, path: str | Path):
        self.path = str(path)
        L = _lib()
        self._L = L
        self._h = L.b200_gguf_open(self.path.encode())
        err = L.b200_gguf_error(self._h)
        if err:
            msg = err.decode()
            L.b200_gguf_close(self._h)
            self._h = None
            raise HartsyInferenceError(f"{self.path}: {msg}")
        self.version = L.b200_gguf_version(self._h)
        self.metadata: dict = json.loads(L.b200_gguf_metadata(self._h).decode("utf-8", errors="replace"))
        self._index = {L.b200_gguf_name(self._h, i).decode(): i for i in range(L.b200_gguf_count(self._h))}
        self.metadata["__has_output_weight__"] = "output.weight" in self._index
        self.metadata["__has_qkv_bias__"] = "blk.0.attn_q.bias" in self._index or "blk.0.attn_qkv.bias" in self._index
        self.metadata["__has_expert_bias__"] = any(k.endswith("exp_probs_b.bias") for k in self._index)

    def keys(self) -> list[str]:
        return list(self._index)

    def __contains__(self, name: str) -> bool:
        return name in self._index

    def info(self, name: str) -> tuple[int, tuple[int, ...]]:
        """(ggml type, shape in row-major order: the last dim is contiguous)."""
        i = self._index[name]
        nd = self._L.b200_gguf_ndim(self._h, i)
        dims = (C.c_int64 * max(nd, 1))()
        self._L.b200_gguf_dims(self._h, i, dims)
        return self._L.b200_gguf_type(self._h, i), tuple(reversed(dims[:nd]))

    def raw(self, name: str) -> torch.Tensor:
        """Packed bytes as stored (zero-copy uint8 view of the mapping)."""
        i = self._index[name]
        n = C.c_uint64()
        ptr = self._L.b200_gguf_data(self._h, i, C.byref(n))
        buf = (C.c_uint8 * n.value).from_address(ptr)
        buf._mapping_owner = self        # storage -> numpy array -> buf -> file: every view keeps the mapping alive
        return torch.from_numpy(np.frombuffer(buf, dtype=np.uint8))

    def get(self, name: str, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        """Dequantised tensor in row-major shape."""
        typ, shape = self.info(name)
        numel = 1
        for s in shape:
            numel *= s
        raw = self.raw(name)
        if typ == 0:
            out = raw.view(torch.float32).reshape(shape)
        elif typ == 1:
            out = raw.view(torch.float16).reshape(shape)
        elif typ == 30:
            out = raw.view(torch.bfloat16).reshape(shape)
        else:
            out = dequantize(raw, typ, numel).reshape(shape)
        return out.to(dtype)

    def close(self) -> None:
        if self._h:
            self._L.b200_gguf_close(self._h)
            self._h = None

    def __del__(self):  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass


# ---------------------------------------------------------------------------------------------
def _w_str(f, s: str) -> None:
    b = s.encode("utf-8")
    f.write(struct.pack("<Q", len(b)))
    f.write(b)


def _w_value(f, v) -> None:
    if isinstance(v, bool):
        f.write(struct.pack("<IB", 7, int(v)))
    elif isinstance(v, int):
        if 0 <= v < 2 ** 32:
            f.write(struct.pack("<II", 4, v))
        else:
            f.write(struct.pack("<Iq", 11, v))
    elif isinstance(v, float):
        f.write(struct.pack("<If", 6, v))
    elif isinstance(v, str):
        f.write(struct.pack("<I", 8))
        _w_str(f, v)
    elif isinstance(v, (list, tuple)):
        f.write(struct.pack("<I", 9))
        if len(v) and isinstance(v[0], str):
            f.write(struct.pack("<IQ", 8, len(v)))
            for s in v:
                _w_str(f, s)
        elif len(v) and isinstance(v[0], float):
            f.write(struct.pack("<IQ", 6, len(v)))
            f.write(np.asarray(v, dtype="<f4").tobytes())
        else:
            f.write(struct.pack("<IQ", 5, len(v)))
            f.write(np.asarray(v, dtype="<i4").tobytes())
    else:
        raise TypeError(f"unsupported GGUF metadata value {type(v)}")


def write_gguf(path: str | Path, metadata: dict, tensors: dict[str, torch.Tensor],
               quant: Optional[dict[str, int] | int] = None, alignment: int = 32) -> None:
    """Write a GGUF v3 file. ``quant`` is a ggml type for every 2-D tensor whose row length fits the
    block size, or a per-name dict; other tensors are stored as F32."""
    names = list(tensors)
    packed: list[tuple[str, tuple[int, ...], int, bytes]] = []
    for name in names:
        t = tensors[name].detach().cpu()
        typ = 0
        if quant is not None:
            want = quant.get(name) if isinstance(quant, dict) else quant
            if want is not None and t.dim() == 2 and t.shape[-1] % type_geometry(want)[0] == 0:
                typ = want
        if typ == 0:
            raw = t.float().contiguous().numpy().tobytes()
        elif typ == 1:
            raw = t.half().contiguous().numpy().tobytes()
        elif typ == 30:
            raw = t.to(torch.bfloat16).contiguous().view(torch.uint8).numpy().tobytes()
        else:
            raw = quantize(t, typ).numpy().tobytes()
        packed.append((name, tuple(t.shape), typ, raw))
    with open(path, "wb") as f:
        md = {k: v for k, v in metadata.items() if not k.startswith("__")}
        md.setdefault("general.alignment", alignment)
        f.write(struct.pack("<IIQQ", 0x46554747, 3, len(packed), len(md)))
        for k, v in md.items():
            _w_str(f, k)
            _w_value(f, v)
        off = 0
        offsets = []
        for name, shape, typ, raw in packed:
            _w_str(f, name)
            f.write(struct.pack("<I", len(shape)))
            for d in reversed(shape):
                f.write(struct.pack("<Q", d))
            f.write(struct.pack("<IQ", typ, off))
            offsets.append(off)
            off += (len(raw) + alignment - 1) // alignment * alignment
        pos = f.tell()
        f.write(b"\0" * ((alignment - pos % alignment) % alignment))
        for (_, _, _, raw) in packed:
            f.write(raw)
            f.write(b"\0" * ((alignment - len(raw) % alignment) % alignment))
