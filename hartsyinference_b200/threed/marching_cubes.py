"""Iso-surface extraction from a scalar grid.

The grid cells are split into six tetrahedra each (marching tetrahedra), which needs no 256-entry
case table: a tetrahedron has only three distinct sign patterns. Vertices on shared edges are
welded by their (sorted) grid-edge key, so the result is a closed, consistently oriented mesh for
a closed iso-surface. The work is vectorised tensor code and runs on CPU or GPU tensors.

Reference behaviour: src/HartsyInference.ThreeD/Geometry/Ops/MarchingCubes.cs (CPU, table-driven
cubes); the surface is the same up to triangulation.
"""
from __future__ import annotations

import torch

# the six tetrahedra of a cube around the 0-6 diagonal; corner i has offset (i&1, (i>>1)&1, (i>>2)&1)
_CORNERS = torch.tensor([[0, 0, 0], [1, 0, 0], [1, 1, 0], [0, 1, 0], [0, 0, 1], [1, 0, 1], [1, 1, 1], [0, 1, 1]])
_TETS = torch.tensor([[0, 5, 1, 6], [0, 1, 2, 6], [0, 2, 3, 6], [0, 3, 7, 6], [0, 7, 4, 6], [0, 4, 5, 6]])


def marching_cubes(volume: torch.Tensor, level: float = 0.0, spacing=(1.0, 1.0, 1.0), origin=(0.0, 0.0, 0.0)):
    """volume [X, Y, Z] -> (vertices float32 [V, 3], faces int64 [F, 3]).

    Inside is ``volume < level``; triangles are wound so that normals point towards larger values
    (outwards for a signed distance field)."""
    v = volume.float()
    dev = v.device
    X, Y, Z = v.shape
    if min(X, Y, Z) < 2:
        return torch.zeros(0, 3), torch.zeros(0, 3, dtype=torch.int64)
    gx, gy, gz = torch.meshgrid(torch.arange(X - 1, device=dev), torch.arange(Y - 1, device=dev),
                                torch.arange(Z - 1, device=dev), indexing="ij")
    base = torch.stack([gx, gy, gz], -1).reshape(-1, 3)                       # [C, 3]
    corners = base[:, None, :] + _CORNERS.to(dev)[None]                        # [C, 8, 3]
    cidx = (corners[..., 0] * Y + corners[..., 1]) * Z + corners[..., 2]       # flat grid index [C, 8]
    vals = v.reshape(-1)[cidx] - level                                         # [C, 8]
    # skip cells that the surface does not cross
    inside = vals < 0
    active = inside.any(1) & (~inside).any(1)
    cidx, vals = cidx[active], vals[active]
    tets = _TETS.to(dev)
    tid = cidx[:, tets].reshape(-1, 4)                                         # [T, 4] grid indices
    tv = vals[:, tets].reshape(-1, 4)
    tin = tv < 0
    n_in = tin.sum(1)
    out_edges = []

    def emit(t_idx, e0, e1, e2, ref):
        """one triangle per selected tetrahedron; e* = (local a, local b) tensors; ref = (grid index
        of an inside corner, grid index of an outside corner) used to orient the triangle"""
        tri = []
        for (a, b) in (e0, e1, e2):
            ia = tid[t_idx, a] if isinstance(a, int) else tid[t_idx].gather(1, a[:, None])[:, 0]
            ib = tid[t_idx, b] if isinstance(b, int) else tid[t_idx].gather(1, b[:, None])[:, 0]
            va = tv[t_idx, a] if isinstance(a, int) else tv[t_idx].gather(1, a[:, None])[:, 0]
            vb = tv[t_idx, b] if isinstance(b, int) else tv[t_idx].gather(1, b[:, None])[:, 0]
            tri.append((ia, ib, va, vb))
        out_edges.append((tri, ref))

    order = torch.argsort(tin.to(torch.int8), dim=1, descending=True, stable=True)   # inside corners first
    for k in (1, 2, 3):
        sel = (n_in == k).nonzero()[:, 0]
        if sel.numel() == 0:
            continue
        o = order[sel]
        p0, p1, p2, p3 = o[:, 0], o[:, 1], o[:, 2], o[:, 3]
        ref = (tid[sel].gather(1, p0[:, None])[:, 0], tid[sel].gather(1, p3[:, None])[:, 0])   # p0 inside, p3 outside
        if k == 1:       # one corner inside: triangle on the three edges leaving it
            emit(sel, (p0, p1), (p0, p2), (p0, p3), ref)
        elif k == 3:     # one corner outside (p3): triangle on the edges reaching it
            emit(sel, (p3, p0), (p3, p2), (p3, p1), ref)
        else:            # two inside (p0, p1), two outside (p2, p3): a quad = two triangles
            emit(sel, (p0, p2), (p0, p3), (p1, p3), ref)
            emit(sel, (p0, p2), (p1, p3), (p1, p2), ref)
    if not out_edges:
        return torch.zeros(0, 3), torch.zeros(0, 3, dtype=torch.int64)
    face_keys, face_ts, ref_in, ref_out = [], [], [], []
    for tri, ref in out_edges:
        ks, ws = [], []
        for (ia, ib, va, vb) in tri:
            lo, hi = torch.minimum(ia, ib), torch.maximum(ia, ib)
            # interpolation weight measured from the lower-index endpoint
            ws.append(torch.where(ia < ib, va / (va - vb), vb / (vb - va)))
            ks.append(lo * (X * Y * Z) + hi)
        face_keys.append(torch.stack(ks, 1))
        face_ts.append(torch.stack(ws, 1))
        ref_in.append(ref[0])
        ref_out.append(ref[1])
    fk = torch.cat(face_keys, 0)
    ft = torch.cat(face_ts, 0)
    uniq, inv = torch.unique(fk.reshape(-1), return_inverse=True)
    faces = inv.reshape(-1, 3)
    # vertex positions from the welded edge keys
    tvals = torch.zeros(uniq.numel(), device=dev)
    tvals[inv] = ft.reshape(-1)
    lo, hi = uniq // (X * Y * Z), uniq % (X * Y * Z)

    def coords(flat):
        return torch.stack([flat // (Y * Z), (flat // Z) % Y, flat % Z], 1).float()

    pos = coords(lo) + (coords(hi) - coords(lo)) * tvals[:, None]
    # orientation: the normal must point from the tetrahedron's inside corner to its outside corner
    outward = coords(torch.cat(ref_out)) - coords(torch.cat(ref_in))
    nrm = torch.cross(pos[faces[:, 1]] - pos[faces[:, 0]], pos[faces[:, 2]] - pos[faces[:, 0]], dim=1)
    flip = (nrm * outward).sum(1) < 0
    faces = torch.where(flip[:, None], faces[:, [0, 2, 1]], faces)
    pos = pos * torch.tensor(spacing, device=dev) + torch.tensor(origin, device=dev)
    # drop degenerate triangles
    ok = (faces[:, 0] != faces[:, 1]) & (faces[:, 1] != faces[:, 2]) & (faces[:, 0] != faces[:, 2])
    return pos.cpu(), faces[ok].cpu()
