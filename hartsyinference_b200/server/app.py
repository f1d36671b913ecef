"""FastAPI application with the reference server's routes.

OpenAI-compatible: ``GET /v1/models``, ``POST /v1/chat/completions`` (SSE streaming with
``data: {json}\\n\\n`` frames and a final ``data: [DONE]``), ``POST /v1/embeddings``,
``POST /v1/images/generations``. Native: ``POST /v1/native/text``, ``/v1/native/text/stream``,
``/v1/native/text/count-tokens``, ``/v1/native/image``, ``/v1/native/video``. Operations:
``/health``, ``/ready`` (reports dead serving loops / unhealthy models), ``/version``, ``/metrics``
(Prometheus), ``/v1/native/admin/free-memory``, ``/v1/native/settings``.
API-key auth (``x-api-key`` or ``Authorization: Bearer``), a per-key rate limiter, usage metering and
a bounded queue that answers 429 when full.

Reference: src/HartsyInference.API/HartsyInferenceServiceExtensions.cs:26-140, Endpoints/
CompatEndpoints.cs:36-258, TextEndpoints.cs, HealthEndpoints.cs:14-20, Metrics.cs, ApiKeyStore,
UsageTracker, HartsyInferenceServerOptions (MaxConcurrency 1, MaxQueueDepth 16).
"""
from __future__ import annotations

import base64
import os
import json
import threading
import time
import uuid
from collections import defaultdict, deque
from dataclasses import dataclass, field
from typing import Optional

import torch
from fastapi import FastAPI, Request
from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse

from .. import __version__
from ..engine.gates import InferenceQueue
from ..engine.inference_engine import InferenceEngine
from ..engine.metrics import REGISTRY
from ..engine.requests import (ChunkKind, EngineOptions, ImageRequest, Modality, ModelSpec, TextRequest, VideoRequest,
                               to_jsonable)
from ..exceptions import HartsyInferenceError, QueueFullError, UnsupportedModelError


@dataclass
class ServerOptions:
    backend: str = "auto"
    max_concurrency: int = 1
    max_queue_depth: int = 16
    api_keys: list[str] = field(default_factory=list)       # empty = auth off
    rate_limit_per_minute: int = 0                          # 0 = unlimited
    models: dict[str, str] = field(default_factory=dict)    # public name -> path / synthetic spec
    allow_model_paths: bool = False                         # let callers name arbitrary local paths as models
    default_text_model: Optional[str] = None
    default_image_model: Optional[str] = None
    default_video_model: Optional[str] = None
    text_max_concurrency: int = 64                          # the text path batches requests itself


class _RateLimiter:
    def __init__(self, per_minute: int):
        self.per_minute = per_minute
        self._hits: dict[str, deque] = defaultdict(deque)
        self._lock = threading.Lock()

    def allow(self, key: str) -> bool:
        if self.per_minute <= 0:
            return True
        now = time.monotonic()
        with self._lock:
            q = self._hits[key]
            while q and now - q[0] > 60.0:
                q.popleft()
            if len(q) >= self.per_minute:
                return False
            q.append(now)
            return True


class UsageTracker:
    def __init__(self):
        self.by_key: dict[str, dict[str, int]] = defaultdict(lambda: defaultdict(int))
        self._lock = threading.Lock()

    def add(self, key: str, **counts: int) -> None:
        with self._lock:
            for k, v in counts.items():
                self.by_key[key][k] += v


def _parse_multipart(body: bytes, content_type: str) -> dict:
    """multipart/form-data -> {field: str | bytes} (file parts keep their bytes)."""
    marker = "boundary="
    if marker not in content_type:
        raise ValueError("multipart body without a boundary")
    boundary = content_type.split(marker, 1)[1].split(";")[0].strip().strip('"').encode()
    out: dict = {}
    for part in body.split(b"--" + boundary):
        part = part.lstrip(b"\r\n")
        if not part or part.startswith(b"--") or b"\r\n\r\n" not in part:
            continue
        head, data = part.split(b"\r\n\r\n", 1)
        data = data[:-2] if data.endswith(b"\r\n") else data
        disp = next((ln for ln in head.decode("utf-8", "replace").split("\r\n") if ln.lower().startswith("content-disposition")), "")
        fields = dict(kv.strip().split("=", 1) for kv in disp.split(";")[1:] if "=" in kv)
        name = fields.get("name", "").strip('"')
        if not name:
            continue
        out[name] = data if "filename" in fields else data.decode("utf-8", "replace")
    return out


def _forced_tool(choice) -> Optional[str]:
    """OpenAI ``tool_choice`` = {"type": "function", "function": {"name": ...}} names the tool to call."""
    if isinstance(choice, dict):
        return (choice.get("function") or {}).get("name")
    return None


def _finish(r) -> str:
    return {"length": "length", "tool_call": "tool_calls"}.get(r.stop_reason.value, "stop")


def _message(r) -> dict:
    m = {"role": "assistant", "content": r.text or (None if r.tool_calls else "")}
    if r.tool_calls:
        m["tool_calls"] = [c.to_openai() for c in r.tool_calls]
    return m


def _flatten_parts(messages: list) -> tuple[list, list]:
    """OpenAI content parts -> plain-text messages ("<image>" where a picture was) + decoded images.
    Only ``data:`` URLs are accepted: the server fetches nothing from the network."""
    import base64
    import io
    out, images = [], []
    for m in messages:
        c = m.get("content")
        if not isinstance(c, list):
            out.append(m)
            continue
        text = ""
        for part in c:
            kind = part.get("type")
            if kind == "text":
                text += part.get("text", "")
            elif kind == "image_url":
                url = (part.get("image_url") or {}).get("url", "")
                if not url.startswith("data:") or "," not in url:
                    raise ValueError("image_url must be a base64 data: URL")
                from PIL import Image
                images.append(Image.open(io.BytesIO(base64.b64decode(url.split(",", 1)[1]))).convert("RGB"))
                text += "<image>\n"
        out.append({**m, "content": text})
    return out, images


def create_app(options: Optional[ServerOptions] = None, engine: Optional[InferenceEngine] = None,
               engine_options: Optional[EngineOptions] = None) -> FastAPI:
    opts = options or ServerOptions()
    eng = engine or InferenceEngine(opts.backend, engine_options)
    app = FastAPI(title="hartsyinference-b200", version=__version__)
    heavy_queue = InferenceQueue(opts.max_concurrency, opts.max_queue_depth)          # image / video
    text_queue = InferenceQueue(opts.text_max_concurrency, opts.max_queue_depth)      # batched by the engine
    limiter = _RateLimiter(opts.rate_limit_per_minute)
    usage = UsageTracker()
    app.state.engine, app.state.usage, app.state.options = eng, usage, opts
    from ..assets.catalog import ModelCacheStore, ModelResolver
    resolver = ModelResolver(store=ModelCacheStore(eng.options.model_cache_directory))

    def resolve(name: Optional[str], modality: Modality) -> ModelSpec:
        default = {Modality.TEXT: opts.default_text_model, Modality.IMAGE: opts.default_image_model,
                   Modality.VIDEO: opts.default_video_model, Modality.EMBEDDINGS: opts.default_text_model}.get(modality)
        name = name or default
        if not name:
            raise UnsupportedModelError("no model named in the request and no default configured")
        path = opts.models.get(name, name)
        if name not in opts.models and not path.startswith("synthetic:"):
            # not a configured name: a catalog id / alias or a repository id that is on disk. A bare
            # filesystem path is honoured only below the model cache directory, or anywhere when the
            # operator opted in (an API caller must not be able to make the server open arbitrary files)
            import os
            real = os.path.realpath(os.path.expanduser(path))
            if os.path.exists(real):
                cache_root = os.path.realpath(os.path.expanduser(eng.options.model_cache_directory))
                inside = real == cache_root or real.startswith(cache_root + os.sep)
                if not (opts.allow_model_paths or inside):
                    raise UnsupportedModelError(f"'{name}' is not a configured model name or catalog id")
                path = real
            else:
                spec = resolver.resolve(path, modality)
                return ModelSpec(requested=spec.local_path or path, modality=modality, catalog=spec.catalog,
                                 local_path=spec.local_path, aux=spec.aux)
        return ModelSpec(requested=path, modality=modality, catalog=name if name in opts.models else None, local_path=path)

    import hmac

    def key_ok(key: str) -> bool:
        # constant-time comparison against every configured key (no early exit on the first match)
        ok = False
        for k in opts.api_keys:
            ok |= hmac.compare_digest(key.encode(), k.encode())
        return ok

    def route_label(request: Request) -> str:
        """The matched route template (bounded label cardinality), not the raw path."""
        for r in app.router.routes:
            try:
                match, _ = r.matches(request.scope)
            except Exception:
                continue
            if match.value == 2:            # starlette.routing.Match.FULL
                return getattr(r, "path", "other")
        return "unmatched"

    @app.middleware("http")
    async def auth_and_metrics(request: Request, call_next):
        path_ = request.url.path
        route = route_label(request)
        key = request.headers.get("x-api-key") or ""
        auth = request.headers.get("authorization", "")
        if not key and auth.lower().startswith("bearer "):
            key = auth[7:].strip()
        open_routes = ("/health", "/ready", "/version", "/metrics", "/openapi.json", "/docs")
        if opts.api_keys and path_ not in open_routes and not key_ok(key):
            REGISTRY.inc("hartsyinference_requests_total", route=route, outcome="unauthorized")
            return JSONResponse({"error": {"message": "invalid or missing API key", "type": "unauthorized"}}, status_code=401)
        if path_ not in open_routes and not limiter.allow(key or request.client.host if request.client else "anon"):
            REGISTRY.inc("hartsyinference_requests_total", route=route, outcome="rate_limited")
            return JSONResponse({"error": {"message": "rate limit exceeded", "type": "rate_limited"}}, status_code=429)
        request.state.api_key = key or "anonymous"
        try:
            resp = await call_next(request)
            outcome = "ok" if resp.status_code < 400 else f"http_{resp.status_code}"
        except Exception:
            outcome = "exception"
            raise
        finally:
            REGISTRY.set("hartsyinference_queue_pending", heavy_queue.pending + text_queue.pending)
        REGISTRY.inc("hartsyinference_requests_total", route=route, outcome=outcome)
        return resp

    @app.exception_handler(QueueFullError)
    async def _queue_full(_, exc):
        return JSONResponse({"error": {"message": str(exc), "type": "queue_full"}}, status_code=429)

    @app.exception_handler(UnsupportedModelError)
    async def _unsupported(_, exc):
        return JSONResponse({"error": {"message": str(exc), "type": "unsupported_model"}}, status_code=400)

    @app.exception_handler(HartsyInferenceError)
    async def _engine_error(_, exc):
        return JSONResponse({"error": {"message": str(exc), "type": type(exc).__name__}}, status_code=500)

    # -------------------------------------------------------------------------- ops routes
    @app.get("/health")
    def health():
        return {"status": "ok"}

    @app.get("/ready")
    def ready():
        bad = eng.unhealthy()
        ranks = eng.ready()          # every rank of a multi-process engine answers through the command stream
        if bad or not all(ranks["healthy"]):
            return JSONResponse({"status": "unhealthy", "models": bad, "ranks": ranks}, status_code=503)
        return {"status": "ready", "backend": eng.backend_description, "loaded": eng.loaded_pipeline_keys, "ranks": ranks}

    @app.get("/version")
    def version():
        return {"version": __version__, "backend": eng.backend_description}

    @app.get("/metrics")
    def metrics():
        return PlainTextResponse(REGISTRY.render(), media_type="text/plain; version=0.0.4")

    @app.post("/v1/native/admin/free-memory")
    def free_memory():
        eng.free_memory()
        return {"status": "freed"}

    @app.get("/v1/native/settings")
    def settings():
        from .. import config
        return {"flags": {f.env: config.get(f.name) for f in config.all_flags()},
                "server": {"max_concurrency": opts.max_concurrency, "max_queue_depth": opts.max_queue_depth}}

    @app.get("/v1/models")
    def models():
        return {"object": "list", "data": [{"id": k, "object": "model", "owned_by": "local"} for k in opts.models]}

    # -------------------------------------------------------------------------- text
    def _text_request(body: dict) -> TextRequest:
        messages, images = _flatten_parts(body.get("messages") or [])
        body = {**body, "messages": messages}
        stop = body.get("stop") or []
        if isinstance(stop, str):
            stop = [stop]
        rf = body.get("response_format") or {}
        return TextRequest(messages=body.get("messages") or [], prompt=body.get("prompt"),
                           temperature=float(body.get("temperature", 0.7)), top_p=float(body.get("top_p", 0.95)),
                           top_k=int(body.get("top_k", 0)), min_p=float(body.get("min_p", 0.0)),
                           repetition_penalty=float(body.get("repetition_penalty", 1.0)),
                           max_tokens=int(body.get("max_tokens") or body.get("max_completion_tokens") or 4096),
                           seed=body.get("seed"), greedy=bool(body.get("greedy", False)) or float(body.get("temperature", 0.7)) == 0.0,
                           enable_thinking=body.get("enable_thinking"), tools=body.get("tools"), stop=list(stop),
                           force_tool_id=_forced_tool(body.get("tool_choice")),
                           json_mode=rf.get("type") == "json_object", images=images)

    @app.post("/v1/chat/completions")
    async def chat_completions(request: Request):
        body = await request.json()
        spec = resolve(body.get("model"), Modality.TEXT)
        treq = _text_request(body)
        rid = "chatcmpl-" + uuid.uuid4().hex[:24]
        created = int(time.time())
        key = request.state.api_key
        if body.get("stream"):
            def gen():
                with text_queue.slot():
                    first = {"id": rid, "object": "chat.completion.chunk", "created": created, "model": body.get("model"),
                             "choices": [{"index": 0, "delta": {"role": "assistant"}, "finish_reason": None}]}
                    yield f"data: {json.dumps(first)}\n\n"
                    for ch in eng.text.stream(spec, treq):
                        if ch.kind == ChunkKind.CHUNK:
                            d = {"id": rid, "object": "chat.completion.chunk", "created": created, "model": body.get("model"),
                                 "choices": [{"index": 0, "delta": {"content": ch.text}, "finish_reason": None}]}
                            yield f"data: {json.dumps(d)}\n\n"
                        elif ch.kind == ChunkKind.RESULT:
                            r = ch.result
                            usage.add(key, prompt_tokens=r.prompt_tokens, completion_tokens=r.completion_tokens)
                            delta = {}
                            if r.tool_calls:
                                delta = {"tool_calls": [{"index": i, **c.to_openai()} for i, c in enumerate(r.tool_calls)]}
                            d = {"id": rid, "object": "chat.completion.chunk", "created": created, "model": body.get("model"),
                                 "choices": [{"index": 0, "delta": delta, "finish_reason": _finish(r)}],
                                 "usage": {"prompt_tokens": r.prompt_tokens, "completion_tokens": r.completion_tokens,
                                           "total_tokens": r.prompt_tokens + r.completion_tokens}}
                            yield f"data: {json.dumps(d)}\n\n"
                    yield "data: [DONE]\n\n"
            return StreamingResponse(gen(), media_type="text/event-stream")
        with text_queue.slot():
            r = eng.text.generate(spec, treq)
        usage.add(key, prompt_tokens=r.prompt_tokens, completion_tokens=r.completion_tokens)
        return {"id": rid, "object": "chat.completion", "created": created, "model": body.get("model"),
                "choices": [{"index": 0, "message": _message(r), "finish_reason": _finish(r)}],
                "usage": {"prompt_tokens": r.prompt_tokens, "completion_tokens": r.completion_tokens,
                          "total_tokens": r.prompt_tokens + r.completion_tokens}}

    @app.post("/v1/native/text")
    async def native_text(request: Request):
        body = await request.json()
        with text_queue.slot():
            r = eng.text.generate(resolve(body.get("model"), Modality.TEXT), _text_request(body))
        return to_jsonable(r)

    @app.post("/v1/native/text/stream")
    async def native_text_stream(request: Request):
        body = await request.json()
        spec, treq = resolve(body.get("model"), Modality.TEXT), _text_request(body)

        def gen():
            with text_queue.slot():
                for ch in eng.text.stream(spec, treq):
                    yield f"data: {json.dumps(to_jsonable(ch))}\n\n"
                yield "data: [DONE]\n\n"
        return StreamingResponse(gen(), media_type="text/event-stream")

    @app.post("/v1/native/text/count-tokens")
    async def count_tokens(request: Request):
        body = await request.json()
        return {"tokens": eng.text.count_tokens(resolve(body.get("model"), Modality.TEXT), _text_request(body))}

    @app.post("/v1/embeddings")
    async def embeddings(request: Request):
        body = await request.json()
        inp = body.get("input")
        texts = [inp] if isinstance(inp, str) else list(inp or [])
        with text_queue.slot():
            emb = eng.embeddings.embed(resolve(body.get("model"), Modality.EMBEDDINGS), texts)
        return {"object": "list", "model": body.get("model"),
                "data": [{"object": "embedding", "index": i, "embedding": e.tolist()} for i, e in enumerate(emb)]}

    # -------------------------------------------------------------------------- audio / vision
    @app.post("/v1/audio/transcriptions")
    async def audio_transcriptions(request: Request):
        import base64
        from ..engine.requests import AudioRequest
        ctype = request.headers.get("content-type", "")
        if ctype.startswith("multipart/form-data"):
            form = _parse_multipart(await request.body(), ctype)
            audio = form.get("file")
        else:
            form = await request.json()
            audio = base64.b64decode(form["audio"]) if form.get("audio") else None
        if not isinstance(audio, (bytes, bytearray)) or not audio:
            return JSONResponse({"error": {"message": "no audio file in the request", "type": "bad_request"}}, status_code=400)
        areq = AudioRequest(audio=bytes(audio), language=form.get("language") or None, task=form.get("task") or "transcribe")
        with heavy_queue.slot():
            res = eng.transcribe.run(resolve(form.get("model"), Modality.TRANSCRIBE), areq)
        if (form.get("response_format") or "json") == "text":
            return PlainTextResponse(res.text)
        out = {"text": res.text}
        if form.get("response_format") == "verbose_json":
            out.update(task=areq.task, language=res.language, duration=res.duration_s,
                       segments=[{"id": i, "start": s.start, "end": s.end, "text": s.text, "tokens": s.tokens,
                                  "avg_logprob": s.avg_logprob, "no_speech_prob": s.no_speech_prob}
                                 for i, s in enumerate(res.segments)])
        return out

    @app.post("/v1/audio/speech")
    async def audio_speech(request: Request):
        from fastapi.responses import Response
        from ..audio import write_wav
        from ..engine.requests import SpeechRequest
        body = await request.json()
        text = body.get("input") or body.get("text") or ""
        if not text.strip():
            return JSONResponse({"error": {"message": "no input text", "type": "bad_request"}}, status_code=400)
        fmt = body.get("response_format") or "wav"
        if fmt not in ("wav", "pcm"):
            return JSONResponse({"error": {"message": f"response_format '{fmt}' is not built (wav, pcm)", "type": "bad_request"}},
                                status_code=400)
        sreq = SpeechRequest(text=text, voice=body.get("voice"), speed=float(body["speed"]) if body.get("speed") else None)
        with heavy_queue.slot():
            res = eng.speech.run(resolve(body.get("model"), Modality.SPEECH), sreq)
        if fmt == "pcm":
            pcm = (res.samples.clamp(-1, 1) * 32767.0).round().to(torch.int16).numpy().tobytes()
            return Response(pcm, media_type="audio/pcm", headers={"x-sample-rate": str(res.sample_rate)})
        return Response(write_wav(None, res.samples, res.sample_rate), media_type="audio/wav")

    @app.post("/v1/native/music")
    async def native_music(request: Request):
        from fastapi.responses import Response
        from ..audio import write_wav
        from ..engine.requests import MusicRequest
        body = await request.json()
        prompt = body.get("prompt") or body.get("input") or ""
        if not prompt.strip():
            return JSONResponse({"error": {"message": "no prompt", "type": "bad_request"}}, status_code=400)
        mreq = MusicRequest(prompt=prompt, seconds=float(body.get("seconds", 5.0)), guidance=float(body.get("guidance", 3.0)),
                            greedy=bool(body.get("greedy", False)), seed=int(body.get("seed", 0)))
        with heavy_queue.slot():
            res = eng.music.run(resolve(body.get("model"), Modality.MUSIC), mreq)
        return Response(write_wav(None, res.samples, res.sample_rate), media_type="audio/wav")

    @app.post("/v1/native/restore")
    async def native_restore(request: Request):
        import io
        from PIL import Image
        from ..engine.requests import RestoreRequest
        body = await request.json()
        raw = body.get("image") or ""
        if not raw:
            return JSONResponse({"error": {"message": "no image", "type": "bad_request"}}, status_code=400)
        b64 = raw.split(",", 1)[1] if raw.startswith("data:") else raw
        img = Image.open(io.BytesIO(base64.b64decode(b64))).convert("RGB")
        rreq = RestoreRequest(operation=body.get("operation", "upscale"), image=img, tile=int(body.get("tile", 128)),
                              tile_overlap=float(body.get("tile_overlap", 0.25)))
        with heavy_queue.slot():
            res = eng.with_vram_cleanup(lambda: eng.restore.run(resolve(body.get("model"), Modality.RESTORE), rreq))
        return {"width": res.width, "height": res.height, "meta": res.meta,
                "png_base64": base64.b64encode(_png(res.rgb, res.width, res.height)).decode()}

    @app.post("/v1/native/mesh")
    async def native_mesh(request: Request):
        import io
        import tempfile
        from PIL import Image
        from ..engine.requests import MeshRequest
        body = await request.json()
        raw = body.get("image") or ""
        if not raw:
            return JSONResponse({"error": {"message": "no image", "type": "bad_request"}}, status_code=400)
        b64 = raw.split(",", 1)[1] if raw.startswith("data:") else raw
        img = Image.open(io.BytesIO(base64.b64decode(b64)))
        fmt = str(body.get("format", "glb")).lower()
        if fmt not in ("glb", "obj", "ply"):
            return JSONResponse({"error": {"message": "format must be glb, obj or ply", "type": "bad_request"}}, status_code=400)
        mreq = MeshRequest(image=img, resolution=int(body.get("resolution", 0)), threshold=body.get("threshold"))
        with heavy_queue.slot():
            res = eng.with_vram_cleanup(lambda: eng.mesh.run(resolve(body.get("model"), Modality.MESH), mreq))
        with tempfile.TemporaryDirectory() as td:
            path = os.path.join(td, "mesh." + fmt)
            res.save(path)
            data = open(path, "rb").read()
        return {"format": fmt, "vertices": len(res.vertices), "faces": len(res.faces), "meta": res.meta,
                "mesh_base64": base64.b64encode(data).decode()}

    def _frame_png(frame) -> str:
        """[3, H, W] float in [0, 1] -> base64 PNG."""
        rgb = (frame.clamp(0, 1) * 255).round().to(torch.uint8).permute(1, 2, 0).contiguous()
        return base64.b64encode(_png(rgb.numpy().tobytes(), rgb.shape[1], rgb.shape[0])).decode()

    def _b64_image(raw: str):
        import io
        from PIL import Image
        b64 = raw.split(",", 1)[1] if raw.startswith("data:") else raw
        return Image.open(io.BytesIO(base64.b64decode(b64)))

    @app.post("/v1/native/world")
    async def native_world(request: Request):
        """Interactive world model. ``{"model", "image"}`` opens a session and returns its id with the
        first frame; ``{"session", "action": [25 floats]}`` advances it by one frame; ``{"session",
        "close": true}`` ends it; ``{"model", "image", "actions": [[...], ...]}`` plays a whole plan."""
        from ..engine.requests import WorldRequest
        body = await request.json()
        world = eng.world
        try:
            if body.get("session") and body.get("close"):
                return {"closed": world.close(body["session"])}
            if body.get("session"):
                with heavy_queue.slot():
                    frame = world.step(body["session"], body.get("action") or [0.0] * 25)
                return {"session": body["session"], "frame_png_base64": _frame_png(frame), "stats": world.stats(body["session"])}
            if not body.get("image"):
                return JSONResponse({"error": {"message": "no image", "type": "bad_request"}}, status_code=400)
            spec = resolve(body.get("model"), Modality.WORLD)
            img = _b64_image(body["image"])
            if body.get("actions") is not None:
                with heavy_queue.slot():
                    res = eng.with_vram_cleanup(lambda: world.run(spec, WorldRequest(image=img, actions=body["actions"], seed=body.get("seed"))))
                return {"frames": len(res.frames), "meta": res.meta, "frames_png_base64": [_frame_png(f) for f in res.frames]}
            with heavy_queue.slot():
                sid, first = world.open(spec, img, int(body.get("seed") or 0))
            return {"session": sid, "frame_png_base64": _frame_png(first)}
        except KeyError as e:
            return JSONResponse({"error": {"message": str(e), "type": "not_found"}}, status_code=404)

    @app.post("/v1/native/vision")
    async def native_vision(request: Request):
        import base64
        import io
        from ..engine.requests import VisionRequest
        body = await request.json()
        images = []
        for im in body.get("images") or []:
            from PIL import Image
            b64 = im.split(",", 1)[1] if im.startswith("data:") else im
            images.append(Image.open(io.BytesIO(base64.b64decode(b64))).convert("RGB"))
        vreq = VisionRequest(operation=body.get("operation", "embed"), images=images, texts=list(body.get("texts") or []),
                             score_threshold=float(body.get("score_threshold", 0.1)), nms_iou=float(body.get("nms_iou", 0.5)),
                             points=list(body.get("points") or []), point_labels=list(body.get("point_labels") or []),
                             boxes=list(body.get("boxes") or []), annotator=str(body.get("annotator", "canny")),
                             canny_low=float(body.get("canny_low", 100.0)), canny_high=float(body.get("canny_high", 200.0)))
        with heavy_queue.slot():
            res = eng.vision.run(resolve(body.get("model"), Modality.VISION), vreq)

        def png(array) -> str:
            import io
            from PIL import Image
            buf = io.BytesIO()
            Image.fromarray(array).save(buf, format="PNG")
            return base64.b64encode(buf.getvalue()).decode()

        if res.control_images is not None:
            return {"control_images": [{"width": int(c.shape[1]), "height": int(c.shape[0]), "png_base64": png(c.numpy())}
                                       for c in res.control_images]}
        if res.labels is not None:
            import numpy as np
            return {"label_maps": [{"width": int(m.shape[1]), "height": int(m.shape[0]), "labels": names,
                                    "png_base64": png(m.numpy().astype(np.uint8 if int(m.max()) < 256 else np.uint16))}
                                   for m, names in zip(res.masks, res.labels)]}
        if res.detections is not None:
            import numpy as np
            for per_image in res.detections:
                for det in per_image:
                    if "mask" in det:                # instance masks travel as 1-bit PNGs
                        mk = det.pop("mask")
                        det["mask_png_base64"] = png((mk.numpy().astype(np.uint8) * 255))
            return {"detections": res.detections}
        if res.masks is not None:
            import io
            import numpy as np
            from PIL import Image
            out_masks = []
            for per_image in res.masks:
                row = []
                for mk in per_image:
                    buf = io.BytesIO()
                    Image.fromarray((mk.clamp(0, 1) * 255).round().numpy().astype(np.uint8)).save(buf, format="PNG")
                    row.append({"width": int(mk.shape[1]), "height": int(mk.shape[0]), "coverage": float((mk > 0.5).float().mean()),
                                "png_base64": base64.b64encode(buf.getvalue()).decode()})
                out_masks.append(row)
            out = {"masks": out_masks}
            if res.mask_scores is not None:
                out["mask_scores"] = [[float(v) for v in sc] for sc in res.mask_scores]
            return out
        if res.depth is not None:
            # 16-bit grayscale PNGs, each map scaled to its own maximum
            import io
            import numpy as np
            from PIL import Image
            maps = []
            for d in res.depth:
                a = (d / d.max().clamp_min(1e-12) * 65535.0).round().numpy().astype(np.uint16)
                buf = io.BytesIO()
                Image.fromarray(a).save(buf, format="PNG")
                maps.append({"width": int(d.shape[1]), "height": int(d.shape[0]), "max": float(d.max()),
                             "png16_base64": base64.b64encode(buf.getvalue()).decode()})
            return {"depth": maps}
        return {k: (v.tolist() if v is not None else None)
                for k, v in (("image_embeddings", res.image_embeddings), ("text_embeddings", res.text_embeddings),
                             ("similarity", res.similarity))}

    # -------------------------------------------------------------------------- image / video
    def _png(rgb: bytes, w: int, h: int) -> bytes:
        from ..utils.png import encode_png
        return encode_png(rgb, w, h)

    @app.post("/v1/images/generations")
    async def images_generations(request: Request):
        body = await request.json()
        size = body.get("size", "1024x1024")
        w, h = (int(v) for v in size.lower().split("x"))
        req = ImageRequest(prompt=body.get("prompt", ""), width=w, height=h, steps=int(body.get("steps", 20)),
                           guidance=float(body.get("guidance", 3.5)), seed=body.get("seed"))
        with heavy_queue.slot():
            res = eng.with_vram_cleanup(lambda: eng.images.generate(resolve(body.get("model"), Modality.IMAGE), req))
        return {"created": int(time.time()), "data": [{"b64_json": base64.b64encode(_png(res.rgb, res.width, res.height)).decode(),
                                                       "seed": res.seed}]}

    @app.post("/v1/native/image")
    async def native_image(request: Request):
        body = await request.json()
        fields = {k: v for k, v in body.items() if k in ImageRequest.__dataclass_fields__}
        for key in ("init_image", "mask_image"):       # base64 (optionally a data: URL); never a server-side path
            if isinstance(fields.get(key), str):
                import io
                from PIL import Image
                b64 = fields[key].split(",", 1)[1] if fields[key].startswith("data:") else fields[key]
                fields[key] = Image.open(io.BytesIO(base64.b64decode(b64))).convert("RGB")
        with heavy_queue.slot():
            res = eng.with_vram_cleanup(lambda: eng.images.generate(resolve(body.get("model"), Modality.IMAGE), ImageRequest(**fields)))
        return {"width": res.width, "height": res.height, "seed": res.seed, "meta": res.meta,
                "png_base64": base64.b64encode(_png(res.rgb, res.width, res.height)).decode()}

    @app.post("/v1/native/video")
    async def native_video(request: Request):
        body = await request.json()
        fields = {k: v for k, v in body.items() if k in VideoRequest.__dataclass_fields__}
        with heavy_queue.slot():
            res = eng.with_vram_cleanup(lambda: eng.video.generate(resolve(body.get("model"), Modality.VIDEO), VideoRequest(**fields)))
        return {"width": res.width, "height": res.height, "fps": res.fps, "seed": res.seed, "meta": res.meta,
                "frames": len(res.frames),
                "first_frame_png_base64": base64.b64encode(_png(res.frames[0], res.width, res.height)).decode() if res.frames else None}

    for route in ("/v1/audio/speech", "/v1/audio/transcriptions", "/v1/native/mesh", "/v1/native/vision",
                  "/v1/native/restore", "/v1/native/world"):
        if any(getattr(r, "path", None) == route for r in app.routes):
            continue
        def _make(r):
            async def _nyi():
                raise UnsupportedModelError(f"{r}: this modality is not built in this engine yet")
            return _nyi
        app.post(route)(_make(route))
    return app
