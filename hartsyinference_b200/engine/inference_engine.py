"""``InferenceEngine``: the public facade.

Mirrors the reference's ``IInferenceEngine`` (src/HartsyInference.Engine/Services/IInferenceEngine.cs:
6-45; InferenceEngine.cs): ``InferenceEngine(backend_selector, options)``, the service properties
(``text``, ``images``, ``video``, ``embeddings``; the remaining modalities raise
``UnsupportedModelError``), ``set_backend``, ``free_memory``, ``is_supported``,
``loaded_pipeline_keys``, and the load / generate wrappers that free cached device memory and retry
once after an out-of-memory error (GenerateWithVramCleanup:224, ConstructWithVramCleanup:270).
Multi-GPU: under ``torch.distributed.run`` every process builds the same engine; rank 0 is the
front, the others call :meth:`InferenceEngine.follow` (the CLI and the server do this), and
``EngineOptions.placement`` decides the process groups (see :mod:`.distributed`; the reference's
EnsureBackend / EnsureCfgParallelBackend / EnsureDitShardBackends / EnsureCpBackends,
InferenceEngine.cs:198-208).
Backend selectors: ``auto | cpu | cuda | cuda:N | cuda:0+cuda:1`` (device lists select multi-GPU
placement); ``vulkan`` is rejected with ``UnsupportedBackendError``
(src/HartsyInference.Engine/BackendFactory.cs).
"""
from __future__ import annotations

import threading
from typing import Callable, Optional, TypeVar

import torch

from .. import log
from ..exceptions import OutOfVramError, UnsupportedBackendError, UnsupportedModelError
from .gates import DeviceGate
from .requests import EngineOptions, Modality

T = TypeVar("T")


def parse_backend_selector(selector: str) -> tuple[str, list[int]]:
    """-> (kind, ordinals). ``auto`` resolves to cuda when a device is present."""
    s = (selector or "auto").strip().lower()
    if s.startswith("vulkan"):
        raise UnsupportedBackendError("the Vulkan backend does not exist in this engine (sm_100a CUDA and CPU only)")
    if s == "auto":
        return ("cuda", [0]) if torch.cuda.is_available() else ("cpu", [])
    if s == "cpu":
        return "cpu", []
    ordinals = []
    for part in s.split("+"):
        part = part.strip()
        if part == "cuda":
            ordinals.append(0)
        elif part.startswith("cuda:"):
            try:
                ordinals.append(int(part[5:]))
            except ValueError:
                raise UnsupportedBackendError(f"bad device ordinal in '{selector}'")
        else:
            raise UnsupportedBackendError(f"unknown backend selector '{selector}'")
    if len(set(ordinals)) != len(ordinals):
        raise UnsupportedBackendError(f"duplicate device in '{selector}'")
    return "cuda", ordinals


class InferenceEngine:
    SUPPORTED = {Modality.TEXT, Modality.IMAGE, Modality.VIDEO, Modality.EMBEDDINGS, Modality.TRANSCRIBE, Modality.VISION, Modality.SPEECH, Modality.RESTORE, Modality.MUSIC, Modality.MESH, Modality.WORLD}

    def __init__(self, backend_selector: str = "auto", options: Optional[EngineOptions] = None, ranks="auto"):
        self.options = options or EngineOptions()
        self.gate = DeviceGate()
        self._services: dict[str, object] = {}
        self._lock = threading.RLock()
        if ranks == "auto":
            from .distributed import RankContext
            ranks = RankContext.from_env()
        self.ranks = ranks
        self.set_backend(backend_selector)
        if self.ranks is not None:
            # every rank owns the services that take part in collective work, so that rank 0's
            # commands find their handlers; followers then wait in follow()
            self.ranks.register("ready", lambda: self.ranks.ready_report(not self.unhealthy()))
            self.ranks.register("release", self._release_local)
            _ = self.text, self.images, self.video

    def follow(self) -> None:
        """Ranks other than 0 of a multi-process engine: execute rank 0's commands until it closes."""
        if self.ranks is not None:
            self.ranks.follow()

    @property
    def is_front(self) -> bool:
        return self.ranks is None or self.ranks.is_front

    def ready(self) -> dict:
        """Health of every rank (``{"ranks": N, "healthy": [...]}``), collected through the command stream."""
        if self.ranks is None:
            return {"ranks": 1, "healthy": [not self.unhealthy()]}
        flags = self.ranks.command("ready")
        return {"ranks": self.ranks.size, "healthy": flags}

    # ------------------------------------------------------------------------------ backend
    def set_backend(self, selector: str) -> None:
        kind, ordinals = parse_backend_selector(selector)
        if kind == "cuda" and not torch.cuda.is_available():
            raise UnsupportedBackendError("no CUDA device is visible")
        if kind == "cuda":
            n = torch.cuda.device_count()
            bad = [o for o in ordinals if o >= n]
            if bad:
                raise UnsupportedBackendError(f"device ordinal(s) {bad} out of range ({n} visible)")
        self.release_loaded()
        self.backend_selector = selector
        self.kind, self.ordinals = kind, ordinals
        self.device = f"cuda:{ordinals[0]}" if kind == "cuda" else "cpu"
        if self.ranks is not None and kind == "cuda":
            # one process per GPU: this process drives the device torchrun gave it
            import os
            local = int(os.environ.get("LOCAL_RANK", "0"))
            self.ordinals = [local]
            self.device = f"cuda:{local}"
        log.decision("Placement", f"backend={self.backend_description}")

    @property
    def backend_description(self) -> str:
        if self.kind == "cpu":
            return "cpu (fp32 oracle path)"
        names = [torch.cuda.get_device_name(o) for o in self.ordinals]
        return f"cuda sm_100a x{len(self.ordinals)}: " + ", ".join(f"cuda:{o} {n}" for o, n in zip(self.ordinals, names))

    def is_supported(self, modality: Modality) -> bool:
        return Modality(modality) in self.SUPPORTED

    # ------------------------------------------------------------------------------ services
    def _service(self, name: str, factory: Callable[[], T]) -> T:
        with self._lock:
            if name not in self._services:
                self._services[name] = factory()
            return self._services[name]  # type: ignore[return-value]

    @property
    def text(self):
        from .text_service import TextService
        return self._service("text", lambda: TextService(self.options, self.device, ranks=self.ranks))

    @property
    def embeddings(self):
        """Encoder checkpoints (BERT family) get their own service; decoder checkpoints are embedded
        by the text service."""
        return _EmbeddingsRouter(self)

    @property
    def images(self):
        from .diffusion_service import ImagesService
        return self._service("images", lambda: ImagesService(self.options, self.device, ranks=self.ranks))

    @property
    def video(self):
        from .diffusion_service import VideoService
        return self._service("video", lambda: VideoService(self.options, self.device, ranks=self.ranks))

    @property
    def transcribe(self):
        from .audio_service import TranscribeService
        return self._service("transcribe", lambda: TranscribeService(self.device))

    @property
    def restore(self):
        from .vision_service import RestoreService
        return self._service("restore", lambda: RestoreService(self.device))

    @property
    def music(self):
        from .audio_service import MusicService
        return self._service("music", lambda: MusicService(self.device))

    @property
    def speech(self):
        from .audio_service import SpeechService
        return self._service("speech", lambda: SpeechService(self.device))

    @property
    def vision(self):
        from .vision_service import VisionService
        return self._service("vision", lambda: VisionService(self.device))

    def _unsupported(self, what: str):
        raise UnsupportedModelError(f"the {what} modality is not built in this engine yet")

    voice_conversion = property(lambda self: self._unsupported("voice conversion"))
    fx = property(lambda self: self._unsupported("fx"))
    @property
    def mesh(self):
        from .mesh_service import MeshService
        return self._service("mesh", lambda: MeshService(self.device))

    @property
    def world(self):
        from .world_service import WorldService
        return self._service("world", lambda: WorldService(self.device))

    # ------------------------------------------------------------------------------ memory
    @property
    def loaded_pipeline_keys(self) -> list[str]:
        keys: list[str] = []
        for s in self._services.values():
            keys += getattr(s, "loaded_keys", lambda: [])()
        return keys

    def release_loaded(self) -> None:
        if getattr(self, "ranks", None) is not None and self.ranks.is_front and self._services:
            self.ranks.command("release")
        else:
            self._release_local()

    def _release_local(self) -> None:
        for s in list(self._services.values()):
            rel = getattr(s, "_release_local", None) or getattr(s, "release", None)
            if rel:
                rel()

    def free_memory(self) -> None:
        """Drop every loaded pipeline and return cached device memory to the driver."""
        self.release_loaded()
        if torch.cuda.is_available():
            torch.cuda.empty_cache()

    def with_vram_cleanup(self, fn: Callable[[], T]) -> T:
        """Run ``fn`` under the device gate; on an out-of-memory error free everything and retry once."""
        ords = self.ordinals or [0]
        with self.gate.acquire(ords):
            try:
                return fn()
            except torch.cuda.OutOfMemoryError as e:
                log.warn(f"[Engine] out of device memory ({e}); freeing loaded pipelines and retrying once")
                self.free_memory()
                try:
                    return fn()
                except torch.cuda.OutOfMemoryError as e2:
                    free, total = torch.cuda.mem_get_info() if torch.cuda.is_available() else (0, 0)
                    raise OutOfVramError(str(e2), requested=0, free=free) from e2

    def unhealthy(self) -> list[str]:
        out: list[str] = []
        for s in self._services.values():
            out += getattr(s, "unhealthy_models", lambda: [])()
        return out

    def close(self) -> None:
        self.release_loaded()
        self._services.clear()
        if self.ranks is not None:
            self.ranks.shutdown()


class _EmbeddingsRouter:
    def __init__(self, engine: "InferenceEngine"):
        self._engine = engine

    def embed(self, spec, texts):
        from .embeddings_service import BertEmbeddingsService, is_bert_dir
        eng = self._engine
        path = spec.local_path or spec.requested
        if is_bert_dir(path):
            svc = eng._service("bert_embeddings", lambda: BertEmbeddingsService(eng.device))
            return svc.embed(spec, texts)
        return eng.text.embed(spec, texts)
