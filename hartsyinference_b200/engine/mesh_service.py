"""Image-to-3-D service: TripoSR checkpoints (a ``.safetensors`` / ``.ckpt`` file or a directory holding
``model.safetensors`` / ``model.ckpt``) -> mesh with vertex colours, written as OBJ / PLY / GLB.

Reference: src/HartsyInference.Engine/Services/MeshService.cs, src/HartsyInference.ThreeD/Pipelines/
TripoSrPipeline.cs (image composited on mid-grey, 512 px, density lattice, marching cubes at 25).
"""
from __future__ import annotations

import threading
import time
from pathlib import Path

import torch

from .. import log
from .requests import MeshRequest, MeshResult, ModelSpec


def prepare_image(image, size: int, foreground_ratio: float = 0.85) -> torch.Tensor:
    """path / PIL image / HWC uint8 array / CHW float tensor (RGB or RGBA) -> [3, size, size] in [0, 1],
    alpha-composited on mid-grey; an RGBA input is first cropped to its opaque region and padded so
    that the object fills ``foreground_ratio`` of the frame."""
    import numpy as np
    if isinstance(image, (str, bytes)) or hasattr(image, "__fspath__"):
        from PIL import Image
        image = Image.open(image)
    if hasattr(image, "convert"):
        image = torch.from_numpy(np.asarray(image.convert("RGBA" if "A" in image.getbands() else "RGB")).copy())
    t = torch.as_tensor(image)
    if t.dtype == torch.uint8:
        t = t.float() / 255.0
    if t.ndim == 3 and t.shape[-1] in (3, 4) and t.shape[0] not in (3, 4):
        t = t.permute(2, 0, 1)
    t = t.float()
    if t.shape[0] == 4:
        rgb, a = t[:3], t[3:4]
        ys, xs = torch.nonzero(a[0] > 0.5, as_tuple=True)
        if ys.numel():
            y0, y1, x0, x1 = int(ys.min()), int(ys.max()) + 1, int(xs.min()), int(xs.max()) + 1
            rgb, a = rgb[:, y0:y1, x0:x1], a[:, y0:y1, x0:x1]
            side = int(max(y1 - y0, x1 - x0) / foreground_ratio)
            py, px = (side - (y1 - y0)) // 2, (side - (x1 - x0)) // 2
            pad = (px, side - (x1 - x0) - px, py, side - (y1 - y0) - py)
            rgb = torch.nn.functional.pad(rgb, pad)
            a = torch.nn.functional.pad(a, pad)
        t = rgb * a + 0.5 * (1 - a)
    t = torch.nn.functional.interpolate(t[None], size=(size, size), mode="bilinear", align_corners=False, antialias=True)[0]
    return t.clamp(0, 1)


class MeshService:
    def __init__(self, device):
        self.device = device
        self._lock = threading.Lock()
        self._loaded: dict = {}

    def loaded_keys(self) -> list[str]:
        return [f"triposr:{k}" for k in self._loaded]

    def release(self) -> None:
        with self._lock:
            self._loaded.clear()

    def _model(self, spec: ModelSpec):
        from ..models.threed.triposr import TRIPOSR, TripoSr, tiny_triposr
        path = spec.local_path or spec.requested
        with self._lock:
            if path not in self._loaded:
                if path.startswith("synthetic:"):
                    cfg = tiny_triposr() if path.endswith("tiny") else TRIPOSR
                    self._loaded[path] = TripoSr(cfg, self.device)
                    return self._loaded[path]
                p = Path(path)
                if p.is_dir():
                    files = sorted(p.glob("*.safetensors")) + sorted(p.glob("*.ckpt")) + sorted(p.glob("*.pth"))
                    if not files:
                        raise ValueError(f"{path}: no .safetensors or .ckpt file")
                    p = files[0]
                if p.suffix == ".safetensors":
                    from ..assets.safetensors import SafeTensorsFile
                    f = SafeTensorsFile(p)
                    tensors = {k: f.get(k) for k in f.keys()}
                else:
                    from ..assets.torch_checkpoint import load_torch_checkpoint
                    tensors = load_torch_checkpoint(p)
                self._loaded[path] = TripoSr(TRIPOSR, self.device, get=tensors.get)
                log.decision("Placement", f"TripoSR on {self.device}: field decode in one kernel per lattice")
            return self._loaded[path]

    def run(self, spec: ModelSpec, req: MeshRequest) -> MeshResult:
        if req.image is None:
            raise ValueError("MeshRequest.image is empty")
        m = self._model(spec)
        t0 = time.perf_counter()
        img = prepare_image(req.image, m.cfg.image_size, req.foreground_ratio)
        planes = m.triplane(img)
        t1 = time.perf_counter()
        verts, faces, rgb = m.extract_mesh(planes, req.resolution or None, req.threshold)
        if str(self.device).startswith("cuda"):
            torch.cuda.synchronize()
        t2 = time.perf_counter()
        res = MeshResult(vertices=verts.cpu(), faces=faces.cpu(), colors=rgb.cpu(),
                         meta={"triplane_s": t1 - t0, "mesh_s": t2 - t1, "resolution": req.resolution or m.cfg.grid_resolution})
        if req.output_path:
            res.save(req.output_path)
        return res
