"""Interactive world models behind ``InferenceEngine.world``: Oasis checkpoints (a DiT ``.safetensors`` /
``.pt`` beside a ViT-VAE one) played frame by frame.

A session holds one world (committed latent frames and their actions). ``open`` encodes the first picture,
``step`` appends the frame that follows one action and returns it, ``close`` frees the session;
``run`` plays a whole list of actions in one call. The model is shared between sessions; a lock per
model keeps their steps apart on the device. Reference: src/HartsyInference.Engine/Services/WorldService.cs,
src/HartsyInference.World/Sessions/ (interactive sessions, frame steppers) and the server's
WorldSessionRegistry."""
from __future__ import annotations

import threading
import time
import uuid
from pathlib import Path
from typing import Optional

import torch

from .. import log
from ..exceptions import UnsupportedModelError as ModelLoadError
from .requests import ModelSpec, WorldRequest, WorldResult

MAX_SESSIONS = 16


def _find(dirpath: Path, needles: tuple) -> Optional[Path]:
    for f in sorted(dirpath.iterdir()):
        if f.suffix in (".safetensors", ".pt", ".pth", ".bin") and any(n in f.name.lower() for n in needles):
            return f
    return None


def _get_from(path: Path):
    if path.suffix == ".safetensors":
        from ..assets.safetensors import SafeTensorsFile
        f = SafeTensorsFile(path)
        keys = set(f.keys())
        return lambda name: f.get(name) if name in keys else None
    from ..assets.torch_checkpoint import load_torch_checkpoint
    return load_torch_checkpoint(path).get


class _Session:
    def __init__(self, world, key: str):
        self.world, self.key = world, key
        self.created = self.touched = time.time()
        self.steps = 0
        self.step_seconds = 0.0


class WorldService:
    def __init__(self, device):
        self.device = device
        self._lock = threading.Lock()
        self._models: dict = {}          # path -> (cfg, dit, vae, model lock)
        self._sessions: dict[str, _Session] = {}

    def loaded_keys(self) -> list[str]:
        return [f"world:{k}" for k in self._models]

    def release(self) -> None:
        with self._lock:
            self._sessions.clear()
            self._models.clear()

    # ------------------------------------------------------------------------------ models
    def _model(self, spec: ModelSpec):
        path = spec.local_path or spec.requested
        with self._lock:
            if path not in self._models:
                from ..models.world.oasis import OasisConfig, OasisDit, OasisVae, tiny_oasis
                if path.startswith("synthetic:oasis"):          # random-init weights of the architecture (benchmarks, tests)
                    cfg = tiny_oasis() if path.endswith(":tiny") else OasisConfig()
                    dit, vae = OasisDit(cfg, self.device, seed=0), OasisVae(cfg, self.device, seed=0)
                else:
                    d = Path(path)
                    if not d.is_dir():
                        raise ModelLoadError(f"{path}: a world model is a directory holding the denoiser and the autoencoder checkpoints")
                    dit_f = _find(d, ("oasis", "dit"))
                    vae_f = _find(d, ("vae", "vit"))
                    if dit_f is None or vae_f is None or dit_f == vae_f:
                        raise ModelLoadError(f"{path}: expected an Oasis denoiser file (name containing 'oasis' or 'dit') and an "
                                             "autoencoder file (name containing 'vae' or 'vit')")
                    cfg = OasisConfig()
                    dit, vae = OasisDit(cfg, self.device, get=_get_from(dit_f)), OasisVae(cfg, self.device, get=_get_from(vae_f))
                log.decision("Placement", f"world model {path}: Oasis DiT depth {cfg.depth} x {cfg.hidden}, window {cfg.max_frames} frames")
                self._models[path] = (cfg, dit, vae, threading.Lock())
            return self._models[path]

    # ------------------------------------------------------------------------------ sessions
    def open(self, spec: ModelSpec, image, seed: int = 0) -> tuple[str, torch.Tensor]:
        """Starts a world from its first picture. Returns (session id, the autoencoder's view of that
        picture [3, H, W] in [0, 1])."""
        from ..models.world.oasis import OasisWorld
        cfg, dit, vae, lk = self._model(spec)
        rgb = self._picture(image, cfg.vae_patch * cfg.patch)
        world = OasisWorld(cfg, dit, vae, seed=seed)
        with lk:
            first = world.reset(rgb)
        sid = uuid.uuid4().hex[:16]
        with self._lock:
            if len(self._sessions) >= MAX_SESSIONS:        # the least recently used session makes room
                old = min(self._sessions, key=lambda k: self._sessions[k].touched)
                del self._sessions[old]
            self._sessions[sid] = _Session(world, spec.local_path or spec.requested)
        return sid, first.float().cpu()

    def step(self, session_id: str, action) -> torch.Tensor:
        """One action [25] (keys / buttons, then the two camera deltas) -> the next frame [3, H, W] in [0, 1]."""
        with self._lock:
            s = self._sessions.get(session_id)
            if s is None:
                raise KeyError(f"no world session '{session_id}'")
            lk = self._models[s.key][3]
        t0 = time.perf_counter()
        with lk:
            frame = s.world.step(torch.as_tensor(action, dtype=torch.float32))
        s.steps += 1
        s.step_seconds += time.perf_counter() - t0
        s.touched = time.time()
        return frame.float().cpu()

    def stats(self, session_id: str) -> dict:
        s = self._sessions[session_id]
        return {"frames": len(s.world.frames), "steps": s.steps,
                "seconds_per_frame": s.step_seconds / s.steps if s.steps else None}

    def close(self, session_id: str) -> bool:
        with self._lock:
            return self._sessions.pop(session_id, None) is not None

    def run(self, spec: ModelSpec, req: WorldRequest) -> WorldResult:
        """First picture + a list of actions -> all frames (the first one included)."""
        sid, first = self.open(spec, req.image, req.seed or 0)
        try:
            frames = [first]
            t0 = time.perf_counter()
            for a in req.actions:
                frames.append(self.step(sid, a))
            dt = time.perf_counter() - t0
        finally:
            self.close(sid)
        return WorldResult(frames=torch.stack(frames), meta={"frames": len(frames), "seconds_per_frame": dt / max(1, len(req.actions))})

    @staticmethod
    def _picture(image, multiple: int) -> torch.Tensor:
        """[3, H, W] in [0, 1] with H, W cut down to multiples of ``multiple``."""
        import numpy as np
        if isinstance(image, (str, bytes)) or hasattr(image, "__fspath__"):
            from PIL import Image
            image = Image.open(image)
        if hasattr(image, "convert"):
            image = torch.from_numpy(np.asarray(image.convert("RGB")).copy())
        t = torch.as_tensor(image)
        if t.dtype == torch.uint8:
            t = t.float() / 255.0
        if t.ndim == 3 and t.shape[-1] == 3 and t.shape[0] != 3:
            t = t.permute(2, 0, 1)
        h, w = t.shape[1] // multiple * multiple, t.shape[2] // multiple * multiple
        if h == 0 or w == 0:
            raise ValueError(f"the first picture must be at least {multiple} x {multiple} pixels")
        return t[:, :h, :w].float().contiguous()
