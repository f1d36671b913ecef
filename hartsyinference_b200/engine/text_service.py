"""Text service: load an LLM once, serve many requests through one continuous-batching loop.

``generate`` blocks, ``stream`` yields ``TextChunk`` records (Chunk ... Result). All requests of a
model share one ``LLMEngine`` driven by a background thread, so concurrent callers are batched
together (in the reference the live routes run one request at a time per device slot and only the
test-hosted ``ModelManager`` batches; src/HartsyInference.Engine/Services/TextService.cs:74-160,
ModelManager.cs:148-212). Prompt-lookup speculative decoding mirrors
``TextGenerationPipeline.GenerateSpeculative`` (n-gram 3, draft 8, look-back 4096;
src/HartsyInference.LLM/Generation/TextGenerationPipeline.cs:403-463) as an n-gram proposer whose
drafts are verified by the engine.
"""
from __future__ import annotations

import contextlib
import queue
import threading
import time
from dataclasses import dataclass, field
from typing import Iterator, Optional

import torch

from .. import config, log
from ..assets.grammar import JsonGrammar
from ..models.llm.loader import LoadedLLM, load_llm
from ..parallel.comm import Comm
from .llm_engine import LLMEngine
from .metrics import REGISTRY
from .requests import ChunkKind, EngineOptions, ModelSpec, StopReason, TextChunk, TextRequest, TextResult
from .sampling import SamplingParams

_REASON = {"stop": StopReason.STOP, "length": StopReason.LENGTH, "cancelled": StopReason.CANCELLED,
           "error": StopReason.ERROR}


@dataclass
class _Hosted:
    llm: LoadedLLM
    engine: LLMEngine
    lock: threading.Lock
    wake: threading.Condition
    thread: Optional[threading.Thread] = None
    running: bool = True
    healthy: bool = True
    key: str = ""
    # SPMD: requests of every replica as seen by rank 0: (replica, request id) -> token callback
    remote_callbacks: Optional[dict] = None
    next_replica: int = 0
    # callers waiting to submit or cancel: the serving loop lets them in between two steps (a Python
    # lock is not fair: a loop that re-acquires it at once would admit waiting callers one at a time)
    waiting_callers: int = 0
    callers_lock: threading.Lock = field(default_factory=threading.Lock)

    @contextlib.contextmanager
    def admitted(self):
        """``with h.admitted():`` = ``with h.wake:`` for callers of the serving loop."""
        with self.callers_lock:
            self.waiting_callers += 1
        try:
            self.wake.acquire()
        finally:
            with self.callers_lock:
                self.waiting_callers -= 1
        try:
            yield
        finally:
            self.wake.release()


class TextService:
    """``ranks`` (an :class:`~hartsyinference_b200.engine.distributed.RankContext`) switches the
    service to SPMD operation: the model is sharded over the placement's tensor-parallel group,
    rank 0 owns the serving loop and broadcasts every scheduler tick (new requests, cancellations,
    "run one step") so that all ranks of a replica step the same batch together; with more replicas
    than one (``dp``), requests are dealt round-robin and each tick gathers the replicas' new tokens
    on rank 0."""

    def __init__(self, options: EngineOptions, device: str = "cuda", comm: Optional[Comm] = None, ranks=None):
        self.options = options
        self.device = device
        self.comm = comm
        self.ranks = ranks
        self.groups = None
        self._models: dict[str, _Hosted] = {}
        self._ssm: dict[str, tuple] = {}
        self._lock = threading.RLock()
        self._tickets: dict[int, object] = {}
        self._next_ticket = 1
        if ranks is not None:
            ranks.register("text.load", self._host_local)
            ranks.register("text.tick", self._tick)
            ranks.register("text.release", self._release_local)

    # ------------------------------------------------------------------------------ loading
    def _key(self, spec: ModelSpec) -> str:
        # the same string on every rank of an SPMD engine (rank 0 names models by it in its commands):
        # the device kind, not the ordinal
        return f"{spec.local_path or spec.requested}|{self.options.placement.cache_key}|{str(self.device).split(':')[0]}"

    def _host(self, spec: ModelSpec) -> _Hosted:
        key = self._key(spec)
        h = self._models.get(key)
        if h is not None:
            return h
        if self.ranks is not None:
            return self.ranks.command("text.load", spec)      # every rank loads its shard
        return self._host_local(spec)

    def _host_local(self, spec: ModelSpec) -> _Hosted:
        path = spec.local_path or spec.requested
        key = self._key(spec)
        with self._lock:
            h = self._models.get(key)
            if h is not None:
                return h
            comm = self.comm
            if self.ranks is not None:
                self.groups = self.ranks.groups(self.options.placement)
                comm = self.groups.inner
            llm = load_llm(path, self.device, comm)
            if comm is not None and comm.world > 1 and llm.model.device.type == "cuda":
                # row-parallel linears through the fused GEMM + all-reduce kernels where they measure faster
                from ..parallel.fused import enable_fused_tp
                try:
                    enable_fused_tp(llm.model, comm, autotune_tokens=min(self.options.max_batch, 64),
                                    large_tokens=int(config.get("prefill_chunk")))
                except Exception as e:
                    log.warn(f"[Collective] fused TP kernels unavailable ({type(e).__name__}: {e}); using NCCL")
            if comm is not None and comm.world > 1 and getattr(llm.model, "dp_attention", False):
                # latent-attention MoE models: decode steps deal the requests over the ranks for attention
                from ..parallel.dp_attention import enable_dp_attention
                enable_dp_attention(llm.model, comm, max_rows=self.options.max_batch)
            eng = LLMEngine(llm.model, page_size=self.options.kv_page_size, max_batch=self.options.max_batch,
                            max_model_len=min(self.options.max_model_len, llm.config.max_position),
                            kv_pool_bytes=self.options.kv_pool_bytes_budget or None)
            eng.on_device_fault = lambda vals, m=llm.model, c=comm: self._on_device_fault(m, c, vals)
            lk = threading.RLock()
            h = _Hosted(llm, eng, lk, threading.Condition(lk), key=key, remote_callbacks={})
            if self.ranks is None or self.ranks.is_front:
                h.thread = threading.Thread(target=self._loop, args=(h,), daemon=True, name=f"llm-loop-{len(self._models)}")
                h.thread.start()
            self._models[key] = h
            return h

    @staticmethod
    def _on_device_fault(model, comm, vals) -> None:
        """A kernel's bounded wait on a peer ran out: leave the peer-memory kernels for NCCL."""
        if comm is not None and comm.world > 1:
            from ..parallel.fused import disable_fused_tp
            log.warn(f"[Collective] device wait timeout {vals}; row-parallel linears fall back to NCCL")
            disable_fused_tp(model, comm)
            ex = getattr(model, "dp_exchange", None)
            if ex is not None and ex.fused:
                from ..parallel.dp_attention import enable_dp_attention
                ex.close()
                enable_dp_attention(model, comm, max_rows=ex.max_rows, fused=False)

    # ------------------------------------------------------------------------------ SPMD ticks
    def _tick(self, key: str, adds: list, cancels: list, step: bool):
        """One scheduler tick, run by every rank with the same arguments. ``adds``: (ticket,
        replica, prompt ids, request, seed, extras); ``cancels``: (replica, request id). Returns, on
        rank 0, ``({ticket: request id}, [(replica, request id, token, finished)])`` for all replicas."""
        h = self._models[key]
        g = self.groups
        mine = g.dp_index if g is not None else 0
        new_ids: dict[int, int] = {}
        for ticket, replica, ids, req, seed, extras in adds:
            if replica != mine:
                continue
            params = self._params(req, h.llm)
            if params.seed is None and not params.is_greedy:
                params.seed = seed               # every rank of the replica must draw the same tokens
            cb = self._tickets.pop(ticket, None) if (self.ranks is None or self.ranks.is_front) else None
            new_ids[ticket] = h.engine.add_request(ids, params, on_token=cb, **(extras or {}))
        for replica, rid in cancels:
            if replica == mine:
                h.engine.cancel(rid)
        events = h.engine.step() if step and h.engine.has_work() else []
        if self.ranks is not None and not self.ranks.is_front:
            for r, _, fin in events:             # nobody collects results on a follower
                if fin:
                    h.engine.release(r)
        if g is None or g.dp <= 1:
            return new_ids, [(mine, r, t, f) for r, t, f in events]
        # replicas other than rank 0's: their leaders report, rank 0 delivers to the callers
        lead = g.inner_rank == 0 and g.cfg_index == 0
        got = self.ranks.gather((mine, new_ids, events) if lead else None)
        if got is None:
            return new_ids, []
        all_ids: dict[int, int] = {}
        all_events = []
        for item in got:
            if item is None:
                continue
            rep, ids_r, ev_r = item
            all_ids.update(ids_r)
            all_events += [(rep, r, t, f) for r, t, f in ev_r]
            if rep != 0:
                for r, t, f in ev_r:
                    cb = h.remote_callbacks.get((rep, r))
                    if cb is not None:
                        cb(r, t, f)
        for ticket, rid in all_ids.items():
            cb = self._tickets.pop(ticket, None)     # tickets of other replicas: remember the caller
            rep = next((a[1] for a in adds if a[0] == ticket), 0)
            if cb is not None and rep != 0:
                h.remote_callbacks[(rep, rid)] = cb
        return all_ids, all_events

    def _submit(self, h: _Hosted, ids: list, req: TextRequest, on_token, extras: dict) -> tuple[int, int]:
        """Queue one request on the engine(s); returns (replica, request id)."""
        if self.ranks is None:
            rid = h.engine.add_request(ids, self._params(req, h.llm), on_token=on_token, **extras)
            return 0, rid
        import random
        with self._lock:
            ticket = self._next_ticket
            self._next_ticket += 1
            self._tickets[ticket] = on_token
        dp = self.groups.dp if self.groups is not None else 1
        replica = h.next_replica % dp
        h.next_replica += 1
        new_ids, _ = self.ranks.command("text.tick", h.key, [(ticket, replica, ids, req, random.getrandbits(31), extras)],
                                        [], False)
        return replica, new_ids[ticket]

    def _cancel(self, h: _Hosted, replica: int, rid: int) -> None:
        if self.ranks is None:
            h.engine.cancel(rid)
        else:
            self.ranks.command("text.tick", h.key, [], [(replica, rid)], False)

    def loaded_keys(self) -> list[str]:
        return list(self._models) + list(self._ssm)

    def unhealthy_models(self) -> list[str]:
        return [k for k, h in self._models.items() if not h.healthy or not (h.thread and h.thread.is_alive())]

    def release(self, key: Optional[str] = None) -> None:
        if self.ranks is not None and self.ranks.is_front and self._models:
            self.ranks.command("text.release", key)
        else:
            self._release_local(key)

    def _release_local(self, key: Optional[str] = None) -> None:
        with self._lock:
            if key is None:
                self._ssm.clear()
            else:
                self._ssm.pop(key, None)
            keys = [key] if key else list(self._models)
            for k in keys:
                h = self._models.pop(k, None)
                if h is None:
                    continue
                with h.wake:
                    h.running = False
                    h.wake.notify_all()
                if h.thread:
                    h.thread.join(timeout=10)
        if torch.cuda.is_available():
            torch.cuda.empty_cache()

    def _loop(self, h: _Hosted) -> None:
        if h.engine.cuda:
            torch.cuda.set_device(h.engine.device)
        while True:
            # callers that want the lock get it before the next step (bounded, so that a stuck caller
            # cannot stop the loop)
            t_yield = time.perf_counter()
            while h.waiting_callers > 0 and h.running and time.perf_counter() - t_yield < 0.05:
                time.sleep(0.0002)
            with h.wake:
                while h.running and not (h.engine.has_work() or h.remote_callbacks):
                    h.wake.wait(timeout=0.5)
                if not h.running:
                    return
                try:
                    if self.ranks is not None:
                        self.ranks.command("text.tick", h.key, [], [], True)
                    else:
                        h.engine.step()
                    st = h.engine.stats()
                    REGISTRY.set("hartsyinference_kv_pages_used", st["pages_used"])
                    REGISTRY.set("hartsyinference_batch_size", st["running"])
                except Exception as e:  # the engine contains step faults itself; this is the last line of defence
                    log.warn(f"[TextService] serving loop error: {type(e).__name__}: {e}")
                    h.healthy = False

    # ------------------------------------------------------------------------------ requests
    def _params(self, req: TextRequest, llm: LoadedLLM) -> SamplingParams:
        mask = None
        if req.json_mode:
            grammar = JsonGrammar(llm.tokenizer)
            mask = grammar.allowed_mask
        return SamplingParams(temperature=req.temperature, top_p=req.top_p, top_k=req.top_k, min_p=req.min_p,
                              repetition_penalty=req.repetition_penalty, max_tokens=req.max_tokens, seed=req.seed,
                              greedy=req.greedy, logits_mask=mask, ignore_eos=req.ignore_eos)

    def count_tokens(self, spec: ModelSpec, req: TextRequest) -> int:
        h = self._host(spec)
        return len(self._prompt_ids(h.llm, req))

    def _prompt_ids(self, llm: LoadedLLM, req: TextRequest) -> list[int]:
        if req.prompt_token_ids is not None:
            return [int(t) for t in req.prompt_token_ids]
        if req.prompt is not None:
            text, special = req.prompt, True
        else:
            text = llm.chat_template.render(req.messages, add_generation_prompt=True, tools=req.tools,
                                            enable_thinking=req.enable_thinking)
            special = not text.startswith(llm.chat_template.bos_token or "\0")
            if req.force_tool_id:
                from ..assets.tool_calls import forced_prefix
                text += forced_prefix(req.force_tool_id)        # the reply is opened as a call of that tool
        if not req.images or llm.vlm is None:
            return llm.tokenizer.encode(text, add_special=special)
        # the text around each "<image>" is tokenised by itself, with the image token id between
        # (Qwen-VL brackets it with its vision-start / vision-end tokens); a prompt with images but no
        # placeholder gets them in front
        marker = [*getattr(llm.vlm, "image_prefix_ids", ()), llm.vlm.image_token_id, *getattr(llm.vlm, "image_suffix_ids", ())]
        if "<image>" not in text:
            text = "<image>" * len(req.images) + text
        ids: list[int] = []
        for i, piece in enumerate(text.split("<image>")):
            if i:
                ids += marker
            if piece:
                ids += llm.tokenizer.encode(piece, add_special=special and i == 0)
        return ids

    def _cross_states(self, llm: LoadedLLM, req: TextRequest):
        """Vision states for a model whose decoder reads images through cross-attention layers
        (Llama 3.2 Vision): the tiles of every image, concatenated. None for other models."""
        if not req.images or llm.vlm is None or not hasattr(llm.vlm, "encode_image"):
            return None
        states = []
        for im in req.images:
            tiles, th, tw = llm.vlm.split_image(self._unit_image(im))
            states.append(llm.vlm.encode_image(tiles, th, tw))
        return torch.cat(states, 0)

    def _multimodal(self, llm: LoadedLLM, req: TextRequest, ids: list[int]):
        """(ids, embeds, mask) with every image token expanded to its patch embeddings."""
        from ..models.encoders.clip_vision import preprocess_image
        if not req.images:
            return ids, None, None
        if llm.vlm is None:
            raise ValueError("this model has no vision tower; images are not accepted")
        if hasattr(llm.vlm, "encode_image"):               # cross-attention models keep one image token per image
            return ids, None, None
        if getattr(llm.vlm, "three_axis_positions", False):   # Qwen-VL: native-resolution patches + three-axis positions
            ids, embeds, mask, pos3, delta = llm.vlm.expand_prompt(ids, [self._unit_image(im) for im in req.images])
            self._mrope = (pos3, delta, llm.vlm.deepstack)
            return ids, embeds, mask
        if hasattr(llm.vlm, "image_features_anyres"):      # any-resolution models take the image at its own size
            return llm.vlm.expand_prompt(ids, [self._unit_image(im) for im in req.images])
        size = llm.vlm.vision.cfg.image_size
        return llm.vlm.expand_prompt(ids, [preprocess_image(im, size) for im in req.images])

    @staticmethod
    def _unit_image(image) -> torch.Tensor:
        """Path, PIL image, uint8 HWC array / tensor or float CHW tensor -> float [3, H, W] in [0, 1]."""
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
        return t.float().clamp(0, 1)

    # ------------------------------------------------------------------------------ recurrent models
    SSM_TYPES = ("mamba", "falcon_mamba", "mamba2", "rwkv", "qwen3_5", "qwen3_5_text", "qwen3_5_moe", "qwen3_5_moe_text")

    def _ssm_kind(self, spec: ModelSpec) -> Optional[str]:
        import json
        from pathlib import Path
        cfg = Path(spec.local_path or spec.requested) / "config.json"
        if not cfg.exists():
            return None
        try:
            mt = json.loads(cfg.read_text()).get("model_type")
        except Exception:
            return None
        return mt if mt in self.SSM_TYPES else None

    def _ssm_host(self, spec: ModelSpec, kind: str):
        """State-space / RWKV checkpoints: a model with constant-size recurrent state instead of a
        paged KV cache (the reference's SsmGenerationPipeline). One request at a time per model."""
        import json
        from pathlib import Path
        from ..assets.chat_template import ChatTemplate
        from ..assets.safetensors import ShardedCheckpoint
        from ..assets.tokenizer import ByteTokenizer, Tokenizer
        from ..models import ssm as S
        path = Path(spec.local_path or spec.requested)
        key = f"ssm|{path}|{self.device}"
        with self._lock:
            if key not in self._ssm:
                raw = json.loads((path / "config.json").read_text())
                get = ShardedCheckpoint(path).get
                if kind in ("mamba", "falcon_mamba"):
                    cfg = S.MambaConfig(bcdt_rms_eps=float(raw.get("mixer_rms_eps", 1e-6)) if kind == "falcon_mamba" else 0.0,
                                        vocab_size=raw["vocab_size"], d_model=raw["hidden_size"], n_layer=raw["num_hidden_layers"],
                                        d_state=raw.get("state_size", 16), d_conv=raw.get("conv_kernel", 4), expand=raw.get("expand", 2),
                                        dt_rank=raw["time_step_rank"] if isinstance(raw.get("time_step_rank"), int) else 0,
                                        rms_eps=raw.get("layer_norm_epsilon", 1e-5), eos_token_id=raw.get("eos_token_id", 0) or 0)
                    model = S.MambaModel(cfg, self.device, get=get)
                elif kind == "mamba2":
                    model = S.Mamba2Model(S.mamba2_from_hf(raw), self.device, get=get)
                elif kind.startswith("qwen3_5"):
                    ck = ShardedCheckpoint(path)
                    nested = ck.get("model.language_model.embed_tokens.weight") is not None     # image-text checkpoints nest the decoder
                    get35 = (lambda n: ck.get(n.replace("model.", "model.language_model.", 1))) if nested else ck.get
                    model = S.Qwen35Model(S.qwen35_from_hf(raw), self.device, get=get35)
                else:
                    model = S.RwkvModel(S.rwkv_from_hf(raw), self.device, get=get)
                tok = Tokenizer.from_hf_json(path / "tokenizer.json") if (path / "tokenizer.json").exists() else \
                    ByteTokenizer(vocab_size=raw["vocab_size"])
                self._ssm[key] = (model, tok, ChatTemplate.for_arch(kind), threading.Lock())
            return self._ssm[key]

    def _stream_ssm(self, spec: ModelSpec, req: TextRequest, kind: str, cancel: Optional[threading.Event]) -> Iterator[TextChunk]:
        from .sampling import sample_row
        model, tok, tpl, lock = self._ssm_host(spec, kind)
        text = req.prompt if req.prompt is not None else tpl.render(req.messages, add_generation_prompt=True)
        ids = tok.encode(text)
        params = SamplingParams(temperature=req.temperature, top_p=req.top_p, top_k=req.top_k, min_p=req.min_p,
                                repetition_penalty=req.repetition_penalty, max_tokens=req.max_tokens, seed=req.seed, greedy=req.greedy)
        gen = torch.Generator(device="cpu").manual_seed(req.seed) if req.seed is not None else None
        t0 = time.perf_counter()
        out_ids: list[int] = []
        out_text, ttft, reason = "", 0.0, StopReason.LENGTH
        dec = tok.stream_decoder()
        with lock:
            state = model.new_state()
            hidden = model.forward(torch.tensor(ids, dtype=torch.int32), state)[-1:]
            for _ in range(req.max_tokens):
                if cancel is not None and cancel.is_set():
                    reason = StopReason.CANCELLED
                    break
                nxt = sample_row(model.logits(hidden)[0].float().cpu(), params, ids + out_ids, gen)
                if not out_ids:
                    ttft = time.perf_counter() - t0
                if nxt == model.cfg.eos_token_id or nxt in getattr(tok, "special_ids", ()):
                    reason = StopReason.STOP
                    break
                out_ids.append(nxt)
                piece = dec.push(nxt)
                if piece:
                    out_text += piece
                    if any(s and s in out_text for s in req.stop):
                        out_text = out_text[: min(out_text.find(s) for s in req.stop if s and s in out_text)]
                        reason = StopReason.STOP
                        break
                    yield TextChunk(ChunkKind.CHUNK, text=piece)
                hidden = model.forward(torch.tensor([nxt], dtype=torch.int32), state)
        res = TextResult(text=out_text, token_ids=out_ids, prompt_tokens=len(ids), completion_tokens=len(out_ids), stop_reason=reason,
                         ttft_s=ttft, total_s=time.perf_counter() - t0)
        yield TextChunk(ChunkKind.STOP_REASON, stop_reason=reason)
        yield TextChunk(ChunkKind.RESULT, result=res)

    def stream(self, spec: ModelSpec, req: TextRequest, cancel: Optional[threading.Event] = None) -> Iterator[TextChunk]:
        kind = self._ssm_kind(spec)
        if kind is not None:
            yield from self._stream_ssm(spec, req, kind, cancel)
            return
        h = self._host(spec)
        llm = h.llm
        ids = self._prompt_ids(llm, req)
        q: "queue.Queue[tuple[int, bool]]" = queue.Queue()
        t0 = time.perf_counter()
        with h.admitted():
            self._mrope = (None, 0, None)
            ids, embeds, emask = self._multimodal(llm, req, ids)
            pos3, delta, deepstack = self._mrope
            replica, rid = self._submit(h, ids, req, lambda r, tok, fin: q.put((tok, fin)),
                                        dict(prompt_embeds=embeds, embeds_mask=emask, cross_states=self._cross_states(llm, req),
                                             positions3=pos3, rope_delta=delta, deepstack=deepstack))
            h.wake.notify_all()
        dec = llm.tokenizer.stream_decoder()
        text = ""
        out_ids: list[int] = []
        ttft = 0.0
        stop_hit = False
        while True:
            if cancel is not None and cancel.is_set():
                with h.admitted():
                    self._cancel(h, replica, rid)
                break
            try:
                tok, fin = q.get(timeout=0.1)
            except queue.Empty:
                if not (h.thread and h.thread.is_alive()):
                    break
                continue
            if tok >= 0:
                if not out_ids:
                    ttft = time.perf_counter() - t0
                out_ids.append(tok)
                piece = dec.push(tok)
                if piece:
                    text += piece
                    cut = min((text.find(s) for s in req.stop if s and s in text), default=-1)
                    if cut >= 0:
                        text = text[:cut]
                        stop_hit = True
                        with h.admitted():
                            self._cancel(h, replica, rid)
                        break
                    yield TextChunk(ChunkKind.CHUNK, text=piece)
            if fin:
                break
        tail = dec.flush()
        if tail and not stop_hit:
            text += tail
            yield TextChunk(ChunkKind.CHUNK, text=tail)
        with h.admitted():
            r = h.engine.release(rid) if replica == (self.groups.dp_index if self.groups is not None else 0) else None
            if h.remote_callbacks is not None:
                h.remote_callbacks.pop((replica, rid), None)
        reason = StopReason.STOP if stop_hit else _REASON.get((r.finish_reason if r else None) or "stop", StopReason.STOP)
        calls = []
        if req.tools or req.force_tool_id:
            from ..assets.tool_calls import forced_prefix, parse_tool_calls, tool_names
            full = (forced_prefix(req.force_tool_id) + text) if req.force_tool_id else text
            cleaned, calls = parse_tool_calls(full, tool_names(req.tools) or None)
            if calls:
                text, reason = cleaned, StopReason.TOOL_CALL
                for c in calls:
                    yield TextChunk(ChunkKind.NATIVE_TOOL_CALL, text=c.arguments, status=c.name)
        res = TextResult(text=text, token_ids=out_ids, prompt_tokens=len(ids), completion_tokens=len(out_ids),
                         stop_reason=reason, ttft_s=ttft, total_s=time.perf_counter() - t0,
                         error=r.error if r else None, tool_calls=calls)
        REGISTRY.inc("hartsyinference_tokens_total", len(out_ids))
        REGISTRY.set("hartsyinference_ttft_seconds", ttft)
        REGISTRY.set("hartsyinference_decode_tok_s", res.tokens_per_second)
        yield TextChunk(ChunkKind.STOP_REASON, stop_reason=reason)
        yield TextChunk(ChunkKind.RESULT, result=res)

    def generate(self, spec: ModelSpec, req: TextRequest, cancel: Optional[threading.Event] = None) -> TextResult:
        res = None
        for ch in self.stream(spec, req, cancel):
            if ch.kind == ChunkKind.RESULT:
                res = ch.result
        assert res is not None
        return res

    def embed(self, spec: ModelSpec, texts: list[str]) -> torch.Tensor:
        """Mean-pooled, L2-normalised final hidden states (decoder-as-embedder, the reference's
        ``DecoderEmbeddingModel``)."""
        from ..models.llm.transformer import ForwardBatch
        h = self._host(spec)
        m = h.llm.model
        outs = []
        with h.wake:
            for t in texts:
                ids = h.llm.tokenizer.encode(t)[: 512]
                n = len(ids)
                dev = m.device
                pages = (n + 15) // 16
                saved = m.kv_cache
                m.alloc_kv(max(pages, 1), 16)
                b = ForwardBatch(tokens=torch.tensor(ids, dtype=torch.int32, device=dev),
                                 positions=torch.arange(n, dtype=torch.int32, device=dev),
                                 slot_mapping=torch.arange(n, dtype=torch.int64, device=dev),
                                 block_table=torch.arange(max(pages, 1), dtype=torch.int32, device=dev)[None],
                                 kv_lens=torch.tensor([n], dtype=torch.int32, device=dev), is_decode=False,
                                 cu_q=torch.tensor([0, n], dtype=torch.int32, device=dev), max_q_len=n, max_kv_len=n)
                hid = m.forward_hidden(b).float().mean(0)
                m.kv_cache = saved
                outs.append(torch.nn.functional.normalize(hid, dim=0).cpu())
        return torch.stack(outs)
