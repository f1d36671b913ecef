"""Mesh and point-cloud writers: Wavefront OBJ, PLY (binary little-endian) and glTF 2.0 binary
(GLB, one mesh with positions, optional normals / vertex colours, uint32 indices).

Reference: src/HartsyInference.ThreeD/Io/GlbWriter.cs, ObjWriter.cs, PlyWriter.cs.
"""
from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np
import torch


def _np(t, dtype):
    return None if t is None else np.ascontiguousarray(torch.as_tensor(t).detach().cpu().numpy().astype(dtype))


def write_obj(path, vertices, faces, normals=None) -> None:
    v, f, n = _np(vertices, np.float32), _np(faces, np.int64), _np(normals, np.float32)
    lines = ["# written by hartsyinference_b200"]
    lines += [f"v {a:.6f} {b:.6f} {c:.6f}" for a, b, c in v]
    if n is not None:
        lines += [f"vn {a:.6f} {b:.6f} {c:.6f}" for a, b, c in n]
        lines += [f"f {a + 1}//{a + 1} {b + 1}//{b + 1} {c + 1}//{c + 1}" for a, b, c in f]
    else:
        lines += [f"f {a + 1} {b + 1} {c + 1}" for a, b, c in f]
    Path(path).write_text("\n".join(lines) + "\n")


def write_ply(path, vertices, faces=None, colors=None) -> None:
    """Binary little-endian PLY; ``colors`` uint8 [V, 3] optional; without faces: a point cloud."""
    v, f, c = _np(vertices, np.float32), _np(faces, np.int32), _np(colors, np.uint8)
    hdr = ["ply", "format binary_little_endian 1.0", f"element vertex {len(v)}",
           "property float x", "property float y", "property float z"]
    if c is not None:
        hdr += ["property uchar red", "property uchar green", "property uchar blue"]
    if f is not None:
        hdr += [f"element face {len(f)}", "property list uchar int vertex_indices"]
    hdr.append("end_header")
    with open(path, "wb") as fh:
        fh.write(("\n".join(hdr) + "\n").encode("ascii"))
        if c is None:
            fh.write(v.tobytes())
        else:
            rec = np.zeros(len(v), dtype=[("p", "<f4", 3), ("c", "u1", 3)])
            rec["p"], rec["c"] = v, c
            fh.write(rec.tobytes())
        if f is not None:
            rec = np.zeros(len(f), dtype=[("n", "u1"), ("i", "<i4", 3)])
            rec["n"], rec["i"] = 3, f
            fh.write(rec.tobytes())


def vertex_normals(vertices, faces) -> torch.Tensor:
    v, f = torch.as_tensor(vertices).float(), torch.as_tensor(faces).long()
    fn = torch.cross(v[f[:, 1]] - v[f[:, 0]], v[f[:, 2]] - v[f[:, 0]], dim=1)
    n = torch.zeros_like(v)
    for k in range(3):
        n.index_add_(0, f[:, k], fn)
    return torch.nn.functional.normalize(n, dim=1)


def write_glb(path, vertices, faces, normals=None, colors=None) -> None:
    v, f = _np(vertices, np.float32), _np(faces, np.uint32)
    n = _np(normals, np.float32)
    c = None if colors is None else _np(torch.as_tensor(colors).float() / (255.0 if torch.as_tensor(colors).dtype == torch.uint8 else 1.0), np.float32)
    chunks, views, accessors, attrs = [], [], [], {}

    def add(arr: np.ndarray, target: int, comp: int, typ: str, minmax: bool = False) -> int:
        off = sum(len(x) for x in chunks)
        raw = arr.tobytes()
        raw += b"\x00" * ((4 - len(raw) % 4) % 4)
        chunks.append(raw)
        views.append({"buffer": 0, "byteOffset": off, "byteLength": arr.nbytes, "target": target})
        acc = {"bufferView": len(views) - 1, "componentType": comp, "count": int(arr.shape[0] if arr.ndim > 1 else arr.size), "type": typ}
        if minmax:
            acc["min"], acc["max"] = arr.min(0).tolist(), arr.max(0).tolist()
        accessors.append(acc)
        return len(accessors) - 1

    attrs["POSITION"] = add(v, 34962, 5126, "VEC3", True)
    if n is not None:
        attrs["NORMAL"] = add(n, 34962, 5126, "VEC3")
    if c is not None:
        attrs["COLOR_0"] = add(c[:, :3], 34962, 5126, "VEC3")
    idx = add(f.reshape(-1), 34963, 5125, "SCALAR")
    binary = b"".join(chunks)
    doc = {"asset": {"version": "2.0", "generator": "hartsyinference_b200"}, "scene": 0, "scenes": [{"nodes": [0]}],
           "nodes": [{"mesh": 0}], "meshes": [{"primitives": [{"attributes": attrs, "indices": idx, "mode": 4}]}],
           "buffers": [{"byteLength": len(binary)}], "bufferViews": views, "accessors": accessors}
    js = json.dumps(doc, separators=(",", ":")).encode("utf-8")
    js += b" " * ((4 - len(js) % 4) % 4)
    total = 12 + 8 + len(js) + 8 + len(binary)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<4sII", b"glTF", 2, total))
        fh.write(struct.pack("<I4s", len(js), b"JSON") + js)
        fh.write(struct.pack("<I4s", len(binary), b"BIN\x00") + binary)
