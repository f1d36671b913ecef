"""safetensors reader (C++ mmap core) and writer, plus the sharded-index loader.

Reader: ``SafeTensorsFile(path)`` maps the file; ``get(name)`` returns a zero-copy CPU tensor over
the mapping. ``ShardedCheckpoint(dir)`` resolves ``model.safetensors.index.json`` or a set of
``*.safetensors`` files to one name -> tensor view. Counterparts: SafeTensorsLoader.Load/GetTensor,
ShardLoader and SafeTensorsWriter (src/HartsyInference.ModelAssets/SafeTensors/).
"""
from __future__ import annotations

import ctypes as C
import json
import struct
from pathlib import Path
from typing import Iterable, Optional

import numpy as np
import torch

from .. import runtime
from ..exceptions import HartsyInferenceError

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool, "F8_E4M3": torch.float8_e4m3fn, "F8_E5M2": torch.float8_e5m2,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafeTensorsFile:
    def __init__(self, path: str | Path):
        self.path = str(path)
        L = runtime.lib()
        self._L = L
        self._h = L.b200_st_open(self.path.encode())
        err = L.b200_st_error(self._h)
        if err:
            msg = err.decode()
            L.b200_st_close(self._h)
            self._h = None
            raise HartsyInferenceError(f"{self.path}: {msg}")
        self._index: dict[str, int] = {}
        for i in range(L.b200_st_count(self._h)):
            self._index[L.b200_st_name(self._h, i).decode()] = i
        self.metadata: dict = json.loads(L.b200_st_metadata(self._h).decode() or "{}")

    def keys(self) -> list[str]:
        return list(self._index)

    def __contains__(self, name: str) -> bool:
        return name in self._index

    def info(self, name: str) -> tuple[str, tuple[int, ...]]:
        i = self._index[name]
        nd = self._L.b200_st_ndim(self._h, i)
        shape = (C.c_int64 * max(nd, 1))()
        self._L.b200_st_shape(self._h, i, shape)
        return self._L.b200_st_dtype(self._h, i).decode(), tuple(shape[:nd])

    def get(self, name: str) -> torch.Tensor:
        """Zero-copy view of the mapped bytes (read-only memory: clone before writing)."""
        i = self._index[name]
        dt, shape = self.info(name)
        nbytes = C.c_uint64()
        ptr = self._L.b200_st_data(self._h, i, C.byref(nbytes))
        if nbytes.value == 0:
            return torch.empty(shape, dtype=_DTYPES[dt])
        buf = (C.c_uint8 * nbytes.value).from_address(ptr)
        # The mapping must outlive every view of these bytes, not just the tensor object returned
        # here: the storage keeps the numpy array, the array keeps ``buf``, and ``buf`` keeps the file.
        buf._mapping_owner = self
        arr = np.frombuffer(buf, dtype=np.uint8)
        return torch.from_numpy(arr).view(_DTYPES[dt]).reshape(shape)

    def close(self) -> None:
        if self._h:
            self._L.b200_st_close(self._h)
            self._h = None

    def __del__(self):  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass


def save_file(tensors: dict[str, torch.Tensor], path: str | Path, metadata: Optional[dict[str, str]] = None) -> None:
    """Write a safetensors file (header JSON padded to 8 bytes, tensors in name order)."""
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    blobs = []
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""   # reshape: scalars have no dim to view
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


class ShardedCheckpoint:
    """Name -> tensor view over a directory (index json or loose shards) or a single file."""

    def __init__(self, path: str | Path):
        p = Path(path)
        self.files: dict[str, SafeTensorsFile] = {}
        self.where: dict[str, str] = {}
        if p.is_file():
            self._add(p)
        else:
            idx = p / "model.safetensors.index.json"
            if not idx.exists():
                cands = sorted(p.glob("*.safetensors.index.json"))
                idx = cands[0] if cands else idx
            if idx.exists():
                wm = json.loads(idx.read_text())["weight_map"]
                for name, fn in wm.items():
                    self.where[name] = fn
                for fn in sorted(set(wm.values())):
                    self.files[fn] = SafeTensorsFile(p / fn)
            else:
                shards = sorted(p.glob("*.safetensors"))
                if not shards:
                    raise HartsyInferenceError(f"no safetensors files under {p}")
                for s in shards:
                    self._add(s)

    def _add(self, f: Path) -> None:
        st = SafeTensorsFile(f)
        self.files[f.name] = st
        for k in st.keys():
            self.where[k] = f.name

    def keys(self) -> Iterable[str]:
        return self.where.keys()

    def get(self, name: str) -> Optional[torch.Tensor]:
        fn = self.where.get(name)
        return None if fn is None else self.files[fn].get(name)

    def metadata(self) -> dict:
        md: dict = {}
        for f in self.files.values():
            md.update(f.metadata)
        return md
