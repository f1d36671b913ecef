"""Continuous-batching LLM engine: paged KV cache, chunked prefill, CUDA-graph decode.

One engine step = ask the C++ scheduler core what to run, fill pinned host buffers with the batch
metadata (token ids, positions, KV slots, block tables, lengths), copy them to the device, run the
prefill chunk batch and/or the decode batch, sample, read the sampled ids back, update requests.

Counterpart in the reference: ``DynamicBatchScheduler`` (SubmitAsync:153, RunLoopAsync:162-268,
AdmitAndPrefill:311-383 prefills each request alone, RunDecodeRound:460-483 gathers pages per
sequence before attention, CaptureGraphSession:397-458 only for a single greedy request;
src/HartsyInference.LLM/Generation/DynamicBatchScheduler.cs), ``TextGenerationPipeline``
(Generate:132-246, GenerateGraphDecode:303-375; src/HartsyInference.LLM/Generation/
TextGenerationPipeline.cs) and ``ModelManager`` (pool sizing ComputeKvPoolPageCount:167;
src/HartsyInference.Engine/ModelManager.cs). Fault containment follows the same rule: an
exception inside a step fails the requests of that step only, the loop stays alive.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Optional, Sequence

import torch

from .. import config, log, ops
from ..exceptions import DeviceWaitTimeout, HartsyInferenceError
from ..models.llm.transformer import DecoderModel, ForwardBatch
from ..ops import _native as N
from ..runtime import KvAllocator, SchedulerCore
from .sampling import SamplingParams, sample_row


@dataclass
class Request:
    id: int
    prompt: list[int]
    params: SamplingParams
    output: list[int] = field(default_factory=list)
    finished: bool = False
    finish_reason: Optional[str] = None     # stop | length | cancelled | error
    on_token: Optional[Callable[[int, int, bool], None]] = None   # (request id, token, finished)
    t_submit: float = 0.0
    t_first_token: float = 0.0
    t_done: float = 0.0
    error: Optional[str] = None
    generator: Optional[torch.Generator] = None
    rng_seed: int = 0                    # stream id of the device sampler (the request's seed, or drawn at submission)
    embeds: Optional[torch.Tensor] = None         # [len(prompt), hidden] replacement input embeddings
    embeds_mask: Optional[torch.Tensor] = None    # [len(prompt)] bool: rows taken from ``embeds``
    cross_states: Optional[torch.Tensor] = None   # [Tv, hidden] vision states read by cross-attention layers
    positions3: Optional[torch.Tensor] = None     # [3, len(prompt)] int32 time / row / column rotary positions (Qwen-VL)
    deepstack: Optional[torch.Tensor] = None      # [taps, len(prompt), hidden] added after the first decoder layers (Qwen3-VL)
    rope_delta: int = 0                           # rotary position of a generated token = its index + rope_delta


def _bucket(n: int) -> int:
    b = 1
    while b < n:
        b *= 2
    return b


class LLMEngine:
    def __init__(self, model: DecoderModel, *, num_pages: Optional[int] = None, page_size: Optional[int] = None,
                 max_batch: Optional[int] = None, prefill_chunk: Optional[int] = None,
                 max_model_len: int = 8192, use_cuda_graphs: Optional[bool] = None,
                 kv_pool_bytes: Optional[int] = None):
        self.model = model
        self.device = model.device
        self.cuda = self.device.type == "cuda"
        self.page = page_size or config.get("kv_page_size")
        self.max_batch = max_batch or config.get("max_batch")
        self.prefill_chunk = prefill_chunk or config.get("prefill_chunk")
        self.max_model_len = max_model_len
        self.max_pages_per_seq = (max_model_len + self.page - 1) // self.page
        self.use_graphs = ((config.get("cuda_graphs") if use_cuda_graphs is None else use_cuda_graphs) and self.cuda
                           and getattr(model.cfg, "graph_safe", True))
        if num_pages is None:
            budget = kv_pool_bytes if kv_pool_bytes is not None else config.get("kv_pool_bytes")
            per_page = model.kv_bytes_per_page(self.page)
            if budget <= 0:
                if self.cuda:
                    free, _ = torch.cuda.mem_get_info(self.device)
                    budget = int(free * 0.85)
                else:
                    budget = 512 << 20      # the reference's default pool budget
            num_pages = max(8, budget // per_page)
            # no point in holding more pages than max_batch full-length sequences can use
            num_pages = min(num_pages, self.max_batch * self.max_pages_per_seq)
        self.num_pages = int(num_pages)
        model.alloc_kv(self.num_pages, self.page)
        self.kv = KvAllocator(self.num_pages, self.page)
        self.sched = SchedulerCore(self.kv, self.max_batch, self.prefill_chunk, 0, cap=max(1024, 2 * self.max_batch))
        self.requests: dict[int, Request] = {}
        self._next_id = 1
        self._graphs: dict[int, tuple] = {}
        self._graphs_disabled = False
        self.fault_injector: Optional[Callable[[str], None]] = None   # host-side test hook
        self.steps = 0
        self.alive = True
        self.h2d_bytes_last = 0
        self.d2h_bytes_last = 0
        self.kernel_launches_last = 0
        self.time_steps = False          # record device time of every step with CUDA events
        self.device_ms_last = 0.0
        self.step_log = None             # a list: every step appends (wall clock at its end, device ms, kernel launches, H2D bytes, D2H bytes, events)
        self._ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) if self.cuda else None
        pin = self.cuda
        mp = self.max_pages_per_seq
        cap_tokens = max(self.prefill_chunk, self.max_batch)
        cap_seqs = max(self.max_batch, 1)
        # pinned host staging, reused every step
        self.h_tokens = torch.zeros(cap_tokens, dtype=torch.int32, pin_memory=pin)
        self.h_positions = torch.zeros(cap_tokens, dtype=torch.int32, pin_memory=pin)
        self.h_slots = torch.zeros(cap_tokens, dtype=torch.int64, pin_memory=pin)
        self.h_table = torch.zeros(cap_seqs, mp, dtype=torch.int32, pin_memory=pin)
        self.h_kv_lens = torch.zeros(cap_seqs, dtype=torch.int32, pin_memory=pin)
        self.h_cu_q = torch.zeros(cap_seqs + 1, dtype=torch.int32, pin_memory=pin)
        self.h_rows = torch.zeros(cap_seqs, dtype=torch.int64, pin_memory=pin)
        self.h_out = torch.zeros(cap_seqs, dtype=torch.int32, pin_memory=pin)
        self.h_status = torch.zeros(4, dtype=torch.int32, pin_memory=pin)
        # called with [code, kernel, site, detail] when a kernel's bounded wait ran out, before the
        # step's requests are failed; a service hangs its fallback (e.g. back to NCCL) here
        self.on_device_fault: Optional[Callable[[list], None]] = None
        if self.cuda:
            N.reserve_workspace(self.device, 256 << 20)
            N.state(self.device).gemm_workspace()
        log.info(f"[Engine] kv pages={self.num_pages} x {self.page} tokens "
                 f"({self.num_pages * model.kv_bytes_per_page(self.page) / 2**30:.2f} GiB), "
                 f"max_batch={self.max_batch}, graphs={'on' if self.use_graphs else 'off'}")

    # ------------------------------------------------------------------------------- requests
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None,
                    on_token: Optional[Callable[[int, int, bool], None]] = None,
                    prompt_embeds: Optional[torch.Tensor] = None, embeds_mask: Optional[torch.Tensor] = None,
                    cross_states: Optional[torch.Tensor] = None, positions3: Optional[torch.Tensor] = None,
                    rope_delta: int = 0, deepstack: Optional[torch.Tensor] = None) -> int:
        """``prompt_embeds`` [len(prompt), hidden] with ``embeds_mask`` [len(prompt)] (bool) replaces the
        token embedding of the marked prompt positions (image patches of a vision-language model).
        ``cross_states`` [Tv, hidden] are the vision states this request's cross-attention layers read
        (Llama 3.2 Vision), during the prefill and every decode step. ``positions3`` [3, len(prompt)]
        gives the prompt's three-axis rotary positions and ``rope_delta`` the offset of every later
        token's rotary position from its sequence index (Qwen-VL image prompts)."""
        params = params or SamplingParams()
        prompt = list(prompt)
        if len(prompt) == 0:
            raise ValueError("empty prompt")
        max_new = min(params.max_tokens, self.max_model_len - len(prompt))
        if max_new <= 0:
            raise ValueError(f"prompt of {len(prompt)} tokens leaves no room (max_model_len={self.max_model_len})")
        rid = self._next_id
        self._next_id += 1
        self.sched.submit(rid, len(prompt), max_new)
        req = Request(rid, prompt, params, on_token=on_token, t_submit=time.perf_counter())
        if prompt_embeds is not None:
            if prompt_embeds.shape[0] != len(prompt):
                raise ValueError("prompt_embeds needs one row per prompt token")
            req.embeds = prompt_embeds.to(self.device).to(torch.bfloat16)
            req.embeds_mask = (embeds_mask if embeds_mask is not None else
                               torch.ones(len(prompt), dtype=torch.bool)).to(self.device)
        if positions3 is not None:
            if positions3.shape != (3, len(prompt)):
                raise ValueError("positions3 needs shape [3, len(prompt)]")
            req.positions3, req.rope_delta = positions3.to(torch.int32).cpu(), int(rope_delta)
        if deepstack is not None:
            if deepstack.shape[1] != len(prompt):
                raise ValueError("deepstack needs one row per prompt token")
            req.deepstack = deepstack.to(self.device).to(torch.bfloat16)
        if cross_states is not None:
            req.cross_states = cross_states.to(self.device).to(torch.bfloat16)
        if params.seed is not None and not params.is_greedy:
            req.generator = torch.Generator(device=self.device).manual_seed(params.seed)
        if params.seed is not None:
            req.rng_seed = int(params.seed) & 0x7fffffff
        else:
            import random
            req.rng_seed = random.getrandbits(31)
        self.requests[rid] = req
        return rid

    def cancel(self, rid: int) -> None:
        req = self.requests.get(rid)
        if req is None or req.finished:
            return
        self.sched.abort(rid)
        self._finish(req, "cancelled")

    def has_work(self) -> bool:
        return any(not r.finished for r in self.requests.values())

    def _finish(self, req: Request, reason: str) -> None:
        req.finished = True
        req.finish_reason = reason
        req.t_done = time.perf_counter()

    # ------------------------------------------------------------------------------- batches
    def _seq_tokens(self, req: Request) -> list[int]:
        return req.prompt + req.output

    def _fill_table(self, row: int, rid: int) -> None:
        self.kv.block_table_into(rid, self.h_table[row].data_ptr(), self.max_pages_per_seq)

    def _to_device(self, t: torch.Tensor, n: int) -> torch.Tensor:
        v = t[:n]
        self.h2d_bytes_last += v.numel() * v.element_size()
        return v.to(self.device, non_blocking=True) if self.cuda else v.clone()

    def _run_prefill(self, chunks: list[tuple[int, int, int]]) -> list[tuple[Request, int]]:
        """Runs one batch of prompt chunks. Returns [(request, sampled token)] for requests whose
        prompt completed in this step."""
        page = self.page
        t = 0
        sample_rows: list[tuple[int, Request]] = []
        max_q = max_kv = 0
        for i, (rid, start, count) in enumerate(chunks):
            req = self.requests[rid]
            toks = self._seq_tokens(req)
            target = len(req.prompt) + len(req.output) - (1 if req.output else 0)
            self.h_tokens[t:t + count] = torch.tensor(toks[start:start + count], dtype=torch.int32)
            self.h_positions[t:t + count] = self._rope_positions(req, start, count)
            self._fill_table(i, rid)
            pos = torch.arange(start, start + count, dtype=torch.int64)
            self.h_slots[t:t + count] = self.h_table[i][(pos // page)].to(torch.int64) * page + pos % page
            self.h_cu_q[i] = t
            self.h_kv_lens[i] = start + count
            max_q = max(max_q, count)
            max_kv = max(max_kv, start + count)
            if start + count >= target:
                sample_rows.append((t + count - 1, req))
            t += count
        n = len(chunks)
        self.h_cu_q[n] = t
        embeds = None
        if any(self.requests[rid].embeds is not None for rid, _, _ in chunks):
            # token embeddings first, then the rows that come from images are overwritten
            cfgm = self.model.cfg
            embeds = ops.embedding(self._to_device(self.h_tokens, t), self.model.embed,
                                    cfgm.embed_scale * cfgm.embedding_multiplier)
            t0 = 0
            for rid, start, count in chunks:
                req = self.requests[rid]
                if req.embeds is not None:
                    end = min(start + count, req.embeds.shape[0])
                    if end > start:
                        m = req.embeds_mask[start:end]
                        rows = embeds[t0:t0 + (end - start)]
                        rows[m] = req.embeds[start:end][m]
                t0 += count
        batch = ForwardBatch(tokens=self._to_device(self.h_tokens, t), positions=self._to_device(self.h_positions, t),
                             slot_mapping=self._to_device(self.h_slots, t), block_table=self._to_device(self.h_table, n),
                             kv_lens=self._to_device(self.h_kv_lens, n), is_decode=False,
                             cu_q=self._to_device(self.h_cu_q, n + 1), max_q_len=max_q, max_kv_len=max_kv,
                             embeds=embeds, cross_states=self._cross_states([self.requests[rid] for rid, _, _ in chunks]),
                             positions3=self._positions3(chunks), deepstack=self._deepstack(chunks, t))
        hidden = self.model.forward_hidden(batch)
        done: list[tuple[Request, int]] = []
        fresh = [(row, req) for row, req in sample_rows if not req.output]
        if fresh:
            rows = torch.tensor([r for r, _ in fresh], dtype=torch.int64)
            rows_d = rows.to(self.device, non_blocking=True) if self.cuda else rows
            self.h2d_bytes_last += rows.numel() * 8
            toks = self._sample(hidden[rows_d].contiguous(), [req for _, req in fresh])
            done = [(req, tok) for (_, req), tok in zip(fresh, toks)]
        # requests that re-computed their context after a pre-emption continue decoding without sampling
        for row, req in sample_rows:
            if req.output:
                done.append((req, -1))
        return done

    def _read_tokens(self, dev_tokens: torch.Tensor, n: int) -> list[int]:
        """Sampled ids and the kernels' status word come back in the same synchronising read. A
        recorded wait timeout (a peer that stopped signalling) fails this step's requests instead
        of letting them continue on garbage."""
        self.h_out[:n].copy_(dev_tokens[:n], non_blocking=True)
        self.h_status.copy_(N.state(self.device).status, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.d2h_bytes_last += n * 4 + 16
        if int(self.h_status[0]) != 0:
            vals = self.h_status.tolist()
            N.state(self.device).reset_after_fault()
            self._graphs.clear()
            if self.on_device_fault is not None:
                self.on_device_fault(vals)
            raise DeviceWaitTimeout(f"device wait failed: code={vals[0]} kernel={vals[1]} site={vals[2]} "
                                    f"detail={vals[3]}", kernel=vals[1], site=vals[2], detail=vals[3])
        return self.h_out[:n].tolist()

    def _sample(self, hidden: torch.Tensor, reqs: list[Request]) -> list[int]:
        """hidden [n, H] for n requests -> one sampled token each."""
        n = len(reqs)
        if all(not r.params.needs_logits for r in reqs):
            tok = self.model.greedy_tokens(hidden)
            if self.cuda:
                return self._read_tokens(tok, n)
            return tok.tolist()
        logits = self.model.full_logits(hidden).float()
        if self.cuda and all(r.params.logits_mask is None for r in reqs):
            return self._sample_on_device(logits, reqs)
        out = []
        for i, r in enumerate(reqs):
            out.append(sample_row(logits[i], r.params, r.prompt + r.output, r.generator))
        self.d2h_bytes_last += n * 4
        return out

    def _sample_on_device(self, logits: torch.Tensor, reqs: list[Request]) -> list[int]:
        """The whole batch in one kernel (temperature -> top-k -> top-p -> min-p -> seeded draw;
        greedy rows are an argmax); repetition penalties are applied to the logits first, also on the
        device. Only the chosen ids come back."""
        n = len(reqs)
        pen = [r for r in reqs if r.params.repetition_penalty != 1.0 and (len(r.prompt) + len(r.output)) > 0]
        if pen:
            width = min(4096, max(len(r.prompt) + len(r.output) for r in pen))
            hist = torch.zeros(n, width, dtype=torch.int32)
            hlen = torch.zeros(n, dtype=torch.int32)
            pv = torch.ones(n, dtype=torch.float32)
            for i, r in enumerate(reqs):
                if r.params.repetition_penalty != 1.0:
                    h = (r.prompt + r.output)[-width:]
                    hist[i, :len(h)] = torch.tensor(h, dtype=torch.int32)
                    hlen[i] = len(h)
                    pv[i] = r.params.repetition_penalty
            ops.repetition_penalty_(logits, hist.to(self.device), hlen.to(self.device), pv.to(self.device))
            self.h2d_bytes_last += hist.numel() * 4 + n * 8
        host = torch.empty(n, 6, dtype=torch.float64)
        for i, r in enumerate(reqs):
            p = r.params
            host[i, 0] = 0.0 if p.is_greedy else max(p.temperature, 1e-6)
            host[i, 1] = p.top_k or 0
            host[i, 2] = p.top_p
            host[i, 3] = p.min_p
            host[i, 4] = r.rng_seed
            host[i, 5] = len(r.output)
        dev = host.to(self.device)
        self.h2d_bytes_last += host.numel() * 8
        tok = ops.sample_tokens(logits, dev[:, 0].float().contiguous(), dev[:, 1].to(torch.int32).contiguous(),
                                dev[:, 2].float().contiguous(), dev[:, 3].float().contiguous(),
                                dev[:, 4].to(torch.int64).contiguous(), dev[:, 5].to(torch.int64).contiguous())
        return self._read_tokens(tok, n)

    def _decode_batch_tensors(self, rids: list[int], bucket: int):
        page = self.page
        n = len(rids)
        max_kv = 0
        for i, rid in enumerate(rids):
            req = self.requests[rid]
            pos = len(req.prompt) + len(req.output) - 1       # position of the token being fed
            self.h_tokens[i] = req.output[-1]
            self.h_positions[i] = pos + req.rope_delta
            self._fill_table(i, rid)
            self.h_slots[i] = int(self.h_table[i, pos // page]) * page + pos % page
            self.h_kv_lens[i] = pos + 1
            max_kv = max(max_kv, pos + 1)
        for i in range(n, bucket):                             # padding rows: no KV write, empty context
            self.h_tokens[i] = 0
            self.h_positions[i] = 0
            self.h_slots[i] = -1
            self.h_kv_lens[i] = 0
            self.h_table[i].zero_()
        return max_kv

    def _run_decode(self, rids: list[int]) -> list[int]:
        n = len(rids)
        reqs = [self.requests[r] for r in rids]
        greedy = all(not r.params.needs_logits for r in reqs)
        if self.use_graphs and greedy and not self._graphs_disabled:
            try:
                return self._run_decode_graph(rids)
            except HartsyInferenceError:
                raise
            except Exception as e:  # capture failure -> circuit breaker, fall back to eager
                self._graphs_disabled = True
                log.warn(f"[Engine] CUDA graph decode disabled after failure: {e}")
        max_kv = self._decode_batch_tensors(rids, n)
        batch = ForwardBatch(tokens=self._to_device(self.h_tokens, n), positions=self._to_device(self.h_positions, n),
                             slot_mapping=self._to_device(self.h_slots, n), block_table=self._to_device(self.h_table, n),
                             kv_lens=self._to_device(self.h_kv_lens, n), is_decode=True, max_kv_len=self.max_model_len,
                             cross_states=self._cross_states(reqs))
        hidden = self.model.forward_hidden(batch)
        return self._sample(hidden, reqs)

    @staticmethod
    def _rope_positions(req: "Request", start: int, count: int) -> torch.Tensor:
        """Rotary positions of sequence rows [start, start + count): the index, shifted by the
        request's offset for rows after the prompt."""
        pos = torch.arange(start, start + count, dtype=torch.int32)
        if req.rope_delta:
            pos = pos + (pos >= len(req.prompt)).to(torch.int32) * req.rope_delta
        return pos

    def _positions3(self, chunks: list) -> Optional[torch.Tensor]:
        """[3, T] rotary positions of a prefill batch when any of its requests carries three-axis
        prompt positions (rows of the other requests repeat their index on all axes)."""
        if not any(self.requests[rid].positions3 is not None for rid, _, _ in chunks):
            return None
        cols = []
        for rid, start, count in chunks:
            req = self.requests[rid]
            p3 = self._rope_positions(req, start, count)[None].expand(3, -1).clone()
            if req.positions3 is not None:
                end = min(start + count, req.positions3.shape[1])
                if end > start:
                    p3[:, :end - start] = req.positions3[:, start:end]
            cols.append(p3)
        return torch.cat(cols, 1).to(self.device)

    def _deepstack(self, chunks: list, total: int) -> Optional[torch.Tensor]:
        """[taps, T, hidden] rows to add after the first decoder layers, for a prefill batch in which
        some request carries them (zero rows elsewhere)."""
        have = [self.requests[rid].deepstack for rid, _, _ in chunks if self.requests[rid].deepstack is not None]
        if not have:
            return None
        out = torch.zeros(max(d.shape[0] for d in have), total, have[0].shape[2], dtype=torch.bfloat16, device=self.device)
        t0 = 0
        for rid, start, count in chunks:
            ds = self.requests[rid].deepstack
            if ds is not None:
                end = min(start + count, ds.shape[1])
                if end > start:
                    out[:ds.shape[0], t0:t0 + end - start] = ds[:, start:end]
            t0 += count
        return out

    @staticmethod
    def _cross_states(reqs: list) -> Optional[list]:
        """One entry per sequence of the batch (None for a request without an image), or None."""
        if not any(r.cross_states is not None for r in reqs):
            return None
        return [r.cross_states for r in reqs]

    def _run_decode_graph(self, rids: list[int]) -> list[int]:
        n = len(rids)
        bucket = min(_bucket(n), _bucket(self.max_batch))
        self._decode_batch_tensors(rids, bucket)
        entry = self._graphs.get(bucket)
        if entry is None:
            entry = self._capture(bucket)
            self._graphs[bucket] = entry
        graph, st, launches = entry
        self.kernel_launches_last += launches
        mp = self.max_pages_per_seq
        st["tokens"].copy_(self.h_tokens[:bucket], non_blocking=True)
        st["positions"].copy_(self.h_positions[:bucket], non_blocking=True)
        st["slots"].copy_(self.h_slots[:bucket], non_blocking=True)
        st["table"].copy_(self.h_table[:bucket], non_blocking=True)
        st["kv_lens"].copy_(self.h_kv_lens[:bucket], non_blocking=True)
        self.h2d_bytes_last += bucket * (4 + 4 + 8 + 4 + 4 * mp)
        graph.replay()
        return self._read_tokens(st["out"], bucket)[:n]

    def _capture(self, bucket: int):
        dev, mp = self.device, self.max_pages_per_seq
        st = {
            "tokens": torch.zeros(bucket, dtype=torch.int32, device=dev),
            "positions": torch.zeros(bucket, dtype=torch.int32, device=dev),
            "slots": torch.full((bucket,), -1, dtype=torch.int64, device=dev),
            "table": torch.zeros(bucket, mp, dtype=torch.int32, device=dev),
            "kv_lens": torch.zeros(bucket, dtype=torch.int32, device=dev),
            "out": torch.zeros(bucket, dtype=torch.int32, device=dev),
        }
        if self.fault_injector is not None:
            self.fault_injector("graph_capture")

        def run():
            batch = ForwardBatch(tokens=st["tokens"], positions=st["positions"], slot_mapping=st["slots"],
                                 block_table=st["table"], kv_lens=st["kv_lens"], is_decode=True,
                                 max_kv_len=self.max_model_len)
            hidden = self.model.forward_hidden(batch)
            self.model.greedy_tokens(hidden, st["out"])

        # warm up on a side stream (loads kernels, sizes scratch) before capturing
        s = torch.cuda.Stream(device=dev)
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            run()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        before = N.launch_count
        with torch.cuda.graph(g):
            run()
        launches = N.launch_count - before
        log.debug(f"[Engine] captured decode graph for batch {bucket} ({launches} kernel launches)")
        return g, st, launches

    # ------------------------------------------------------------------------------- step loop
    def step(self) -> list[tuple[int, int, bool]]:
        """One engine iteration. Returns [(request id, new token, finished)]."""
        self.h2d_bytes_last = 0
        self.d2h_bytes_last = 0
        self.kernel_launches_last = 0
        launches_before = N.launch_count
        if self.time_steps and self.cuda:
            self._ev[0].record()
        prefill, decode, preempted = self.sched.step()
        for rid in preempted:
            log.debug(f"[Engine] request {rid} pre-empted (KV pool full), will recompute")
        events: list[tuple[int, int, bool]] = []
        involved = [rid for rid, _, _ in prefill] + list(decode)
        try:
            if self.fault_injector is not None:
                self.fault_injector("step")
            new_tokens: dict[int, int] = {}
            if decode:
                toks = self._run_decode(decode)
                for rid, tok in zip(decode, toks):
                    new_tokens[rid] = tok
            completed_prefill: list[tuple[Request, int]] = []
            if prefill:
                completed_prefill = self._run_prefill(prefill)
            done_ids = {req.id for req, _ in completed_prefill}
            for rid, _, _ in prefill:
                if rid not in done_ids:
                    self.sched.update(rid, 0, False)        # partial chunk: nothing sampled yet
            for req, tok in completed_prefill:
                if tok < 0:
                    self.sched.update(req.id, 0, False)     # context rebuilt after pre-emption
                else:
                    new_tokens[req.id] = tok
            now = time.perf_counter()
            for rid, tok in new_tokens.items():
                req = self.requests[rid]
                if req.finished:
                    continue
                req.output.append(tok)
                if len(req.output) == 1:
                    req.t_first_token = now
                p = req.params
                stop = (not p.ignore_eos and tok in self.model.cfg.eos_token_ids) or tok in p.stop_token_ids
                limit = len(req.output) >= min(p.max_tokens, self.max_model_len - len(req.prompt))
                fin = stop or limit
                self.sched.update(rid, 1, fin)
                if fin:
                    self._finish(req, "stop" if stop else "length")
                events.append((rid, tok, fin))
                if req.on_token is not None:
                    req.on_token(rid, tok, fin)
        except Exception as e:
            # fault containment: fail the requests of this step, keep the loop alive
            log.warn(f"[Engine] step failed ({type(e).__name__}: {e}); failing {len(involved)} request(s)")
            for rid in involved:
                req = self.requests.get(rid)
                if req is not None and not req.finished:
                    self.sched.abort(rid)
                    req.error = f"{type(e).__name__}: {e}"
                    self._finish(req, "error")
                    events.append((rid, -1, True))
                    if req.on_token is not None:
                        req.on_token(rid, -1, True)
        self.steps += 1
        self.kernel_launches_last += N.launch_count - launches_before
        if self.time_steps and self.cuda:
            self._ev[1].record()
            self._ev[1].synchronize()
            self.device_ms_last = self._ev[0].elapsed_time(self._ev[1])
        if self.step_log is not None:
            self.step_log.append((time.perf_counter(), self.device_ms_last, self.kernel_launches_last, self.h2d_bytes_last,
                                  self.d2h_bytes_last, len(events)))
        return events

    def run_until_done(self, max_steps: int = 1 << 30) -> None:
        n = 0
        while self.has_work() and n < max_steps:
            self.step()
            n += 1

    def generate(self, prompts: Sequence[Sequence[int]], params: Optional[SamplingParams] = None) -> list[list[int]]:
        """Blocking convenience call: submit all prompts, run to completion, return the generated ids."""
        ids = [self.add_request(p, params) for p in prompts]
        self.run_until_done()
        outs = [self.requests[i].output for i in ids]
        return outs

    def release(self, rid: int) -> Optional[Request]:
        return self.requests.pop(rid, None)

    def stats(self) -> dict:
        s = self.sched.stats()
        s.update(steps=self.steps, pages=self.num_pages, pages_used=self.num_pages - s["free_blocks"],
                 graphs=len(self._graphs), alive=self.alive)
        return s
