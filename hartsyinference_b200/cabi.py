"""Python side of the C ABI (``libb200infer.so``): owns the engine objects, speaks JSON.

Every function returns ``(code, message, payload)``; the C layer turns that into return codes,
``b200_last_error`` and out-parameters. Callbacks arrive as raw function-pointer integers."""
from __future__ import annotations

import ctypes as C
import json
import threading
from typing import Any

from .engine.inference_engine import InferenceEngine
from .engine.requests import (ChunkKind, EngineOptions, ImageRequest, Modality, ModelSpec, TextRequest, VideoRequest,
                              to_jsonable)
from .exceptions import HartsyInferenceError, RequestCancelled
from .parallel.config import ParallelConfig

_engines: dict[int, InferenceEngine] = {}
_next = [1]
_lock = threading.Lock()

CHUNK_CB = C.CFUNCTYPE(C.c_int, C.c_char_p, C.c_char_p, C.c_void_p)
STEP_CB = C.CFUNCTYPE(C.c_int, C.c_int, C.c_int, C.c_void_p)


def _guard(fn):
    def wrapped(*a):
        try:
            return 0, "", fn(*a)
        except HartsyInferenceError as e:
            return getattr(e, "code", 1), f"{type(e).__name__}: {e}", None
        except Exception as e:  # noqa: BLE001 - the C caller gets a code + message, never an exception
            return 1, f"{type(e).__name__}: {e}", None
    wrapped.__name__ = fn.__name__
    return wrapped


def _spec(js: str) -> ModelSpec:
    d = json.loads(js) if js else {}
    if isinstance(d, str):
        d = {"requested": d}
    return ModelSpec(requested=d.get("requested") or d.get("Requested") or d.get("local_path") or "",
                     modality=Modality(d.get("modality", d.get("Modality", "text")).lower()),
                     catalog=d.get("catalog"), local_path=d.get("local_path") or d.get("LocalPath"),
                     aux=d.get("aux") or d.get("Aux") or {})


def _fields(cls, js: str) -> Any:
    d = json.loads(js) if js else {}
    low = {k[0].lower() + k[1:] if k and k[0].isupper() else k: v for k, v in d.items()}
    # accept PascalCase (the .NET facade serialises its records as-is) and snake_case
    snake = {}
    for k, v in low.items():
        s = "".join("_" + c.lower() if c.isupper() else c for c in k)
        snake[s] = v
    return cls(**{k: v for k, v in snake.items() if k in cls.__dataclass_fields__})


@_guard
def engine_create(selector: str, options_json: str) -> int:
    d = json.loads(options_json or "{}")
    opts = EngineOptions()
    for k, v in d.items():
        k2 = "".join("_" + c.lower() if c.isupper() else c for c in k).lstrip("_")
        if k2 == "placement" and isinstance(v, str):
            opts.placement = ParallelConfig.parse(v)
        elif hasattr(opts, k2) and k2 != "placement":
            setattr(opts, k2, v)
    eng = InferenceEngine(selector, opts)
    with _lock:
        h = _next[0]
        _next[0] += 1
        _engines[h] = eng
    return h


@_guard
def engine_destroy(h: int) -> None:
    eng = _engines.pop(h, None)
    if eng is not None:
        eng.close()


@_guard
def engine_set_backend(h: int, selector: str) -> None:
    _engines[h].set_backend(selector)


@_guard
def engine_describe(h: int) -> str:
    e = _engines[h]
    return json.dumps({"backend_selector": e.backend_selector, "backend_description": e.backend_description,
                       "loaded_pipeline_keys": e.loaded_pipeline_keys})


@_guard
def engine_is_supported(h: int, modality: str) -> bool:
    try:
        return _engines[h].is_supported(Modality(modality.lower()))
    except ValueError:
        return False


@_guard
def free_memory(h: int) -> None:
    _engines[h].free_memory()


@_guard
def text_generate(h: int, spec: str, req: str) -> str:
    r = _engines[h].text.generate(_spec(spec), _fields(TextRequest, req))
    return json.dumps(to_jsonable(r))


@_guard
def text_stream(h: int, spec: str, req: str, cb_ptr: int, user: int) -> None:
    cb = CHUNK_CB(cb_ptr)
    cancel = threading.Event()
    for ch in _engines[h].text.stream(_spec(spec), _fields(TextRequest, req), cancel):
        if ch.kind == ChunkKind.CHUNK:
            payload = ch.text
        elif ch.kind == ChunkKind.RESULT:
            payload = json.dumps(to_jsonable(ch.result))
        elif ch.kind == ChunkKind.STOP_REASON:
            payload = ch.stop_reason.value
        else:
            payload = ch.status or ""
        if cb(ch.kind.value.encode(), payload.encode("utf-8"), user) != 0:
            cancel.set()


@_guard
def text_count_tokens(h: int, spec: str, req: str) -> int:
    return _engines[h].text.count_tokens(_spec(spec), _fields(TextRequest, req))


def _step_adapter(cb_ptr: int, user: int):
    if not cb_ptr:
        return None
    cb = STEP_CB(cb_ptr)

    def on_step(p):
        if cb(p.step, p.total_steps, user) != 0:
            raise RequestCancelled("cancelled by the step callback")
    return on_step


@_guard
def image_generate(h: int, spec: str, req: str, cb_ptr: int, user: int):
    e = _engines[h]
    r = e.with_vram_cleanup(lambda: e.images.generate(_spec(spec), _fields(ImageRequest, req), _step_adapter(cb_ptr, user)))
    return (r.rgb, r.width, r.height, r.seed)


@_guard
def video_generate(h: int, spec: str, req: str, cb_ptr: int, user: int):
    e = _engines[h]
    r = e.with_vram_cleanup(lambda: e.video.generate(_spec(spec), _fields(VideoRequest, req), _step_adapter(cb_ptr, user)))
    return (b"".join(r.frames), len(r.frames), r.width, r.height, r.fps, r.seed)


@_guard
def transcribe(h: int, spec: str, req: str, pcm: bytes, sample_rate: int):
    import numpy as np
    import torch
    from .engine.requests import AudioRequest
    e = _engines[h]
    r = _fields(AudioRequest, req)
    r.audio = torch.from_numpy(np.frombuffer(pcm, dtype="<f4").copy())
    r.sample_rate = sample_rate
    res = e.transcribe.run(_spec(spec), r)
    return json.dumps({"text": res.text, "language": res.language, "duration": res.duration_s,
                       "segments": [{"start": s.start, "end": s.end, "text": s.text} for s in res.segments]})


@_guard
def speak(h: int, spec: str, req: str):
    from .engine.requests import SpeechRequest
    e = _engines[h]
    res = e.speech.run(_spec(spec), _fields(SpeechRequest, req))
    return (res.samples.float().contiguous().numpy().astype("<f4").tobytes(), res.sample_rate)


@_guard
def music(h: int, spec: str, req: str):
    from .engine.requests import MusicRequest
    e = _engines[h]
    res = e.music.run(_spec(spec), _fields(MusicRequest, req))
    return (res.samples.float().contiguous().numpy().astype("<f4").tobytes(), res.sample_rate)


@_guard
def embed_text(h: int, spec: str, texts: str):
    e = _engines[h]
    s = _spec(spec)
    s.modality = Modality.EMBEDDINGS
    emb = e.embeddings.embed(s, list(json.loads(texts)))
    return (emb.float().contiguous().numpy().astype("<f4").tobytes(), int(emb.shape[0]), int(emb.shape[1]))


def _rgb(buf: bytes, width: int, height: int):
    import numpy as np
    import torch
    return torch.from_numpy(np.frombuffer(buf, dtype=np.uint8).reshape(height, width, 3).copy())


@_guard
def embed_image(h: int, spec: str, rgb: bytes, width: int, height: int):
    from .engine.requests import VisionRequest
    e = _engines[h]
    res = e.vision.run(_spec(spec), VisionRequest(images=[_rgb(rgb, width, height)]))
    v = res.image_embeddings[0].float().contiguous()
    return (v.numpy().astype("<f4").tobytes(), int(v.numel()))


@_guard
def upscale(h: int, spec: str, req: str, rgb: bytes, width: int, height: int):
    from .engine.requests import RestoreRequest
    e = _engines[h]
    r = _fields(RestoreRequest, req)
    r.image = _rgb(rgb, width, height)
    res = e.with_vram_cleanup(lambda: e.restore.run(_spec(spec), r))
    return (res.rgb, res.width, res.height)
