"""Fused compute + collective paths for tensor parallelism.

``FusedRowParallel`` runs the row-parallel linears of a TP group (attention output projection,
FFN down projection) as ONE kernel per linear (``b200_gemm_allreduce``,
csrc/kernels/gemm_tcgen05.cu): tcgen05 GEMM tiles of the rank's partial product are stored into
the rank's own part of the symmetric heap; each rank then pulls the token rows it owns summed over
all ranks (``multimem.ld_reduce``: the NVSwitch adds the copies; peer loads when the heap has no
multicast mapping), adds the residual row, applies the RMSNorm that follows the linear, optionally
quantises to e4m3 for the next linear, and stores the result into every rank (``multimem.st``).
So the all-reduce, the residual add, the norm and the activation quantisation of the next GEMM
are the epilogue of the GEMM. It covers token counts up to 128 (the decode regime, where the
all-reduce is latency-bound); larger batches use the plain GEMM and an NCCL all-reduce, which is
also the measured baseline of the fused path.

The reference performs the same two reductions per layer with ``AllReduceSum`` after the o-proj and
the down-proj (src/HartsyInference.LLM/Transformer/TensorParallelTransformer.cs:298,307) through
NCCL calls issued by one thread for all ranks (src/HartsyInference.Cuda/NcclComm.cs:53-85), and
runs the residual add + norm as separate kernels afterwards.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from .. import config, log, ops
from ..ops import Fp8Act, LinearWeight
from ..ops import _native as N
from .comm import Comm
from .symm import SymmetricHeap

MAX_TOKENS = 128
PART_SPLITS = 4       # K splits per rank that the partial buffer has room for
LARGE_SLOTS = 4       # output buffers of the > 128-token form (the caller names the one to write)


class FusedRowParallel:
    def __init__(self, comm: Comm, max_features: int, device: Optional[torch.device] = None,
                 num_out_buffers: int = 2, emulate_peers: bool = False, max_large_tokens: int = 0):
        """``emulate_peers`` (measurement aid for one GPU): ``comm`` claims a rank of a larger world
        but has no peers; every "peer" address is this GPU's own buffer, so the kernel runs the full
        protocol of that rank (its row share, one signal per pretended peer) with meaningless sums."""
        self.comm = comm
        self.rank, self.world = comm.rank, comm.world
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        heap_comm = comm
        if emulate_peers:
            from .comm import SingleComm
            heap_comm = SingleComm()
        self.max_features = max_features
        f = max_features
        part_bytes = PART_SPLITS * MAX_TOKENS * f * 2
        bf16_bytes = MAX_TOKENS * f * 2
        q_bytes = MAX_TOKENS * f
        sf_bytes = max(MAX_TOKENS * ((f + 127) // 128) * 4, ((f + 511) // 512) * 512)
        per_slot = bf16_bytes + q_bytes + sf_bytes + 3 * 256
        # sequences of more than MAX_TOKENS rows (prefill, DiT): one [tokens][features] partial buffer
        # and two output buffers
        self.max_large_tokens = int(max_large_tokens)
        large_bytes = self.max_large_tokens * f * 2
        self.heap = SymmetricHeap(heap_comm, part_bytes + num_out_buffers * per_slot + (LARGE_SLOTS + 1) * (large_bytes + 256) + 16384, self.device)
        self.use_mc = self.heap.has_multicast
        self.off_part = self.heap.alloc(part_bytes)
        self.off_bf16 = [self.heap.alloc(bf16_bytes) for _ in range(num_out_buffers)]
        self.off_q = [self.heap.alloc(q_bytes) for _ in range(num_out_buffers)]
        self.off_sf = [self.heap.alloc(sf_bytes) for _ in range(num_out_buffers)]
        self.off_part_large = self.heap.alloc(large_bytes) if large_bytes else 0
        self.off_out_large = [self.heap.alloc(large_bytes) for _ in range(LARGE_SLOTS)] if large_bytes else []
        self.off_flags = self.heap.alloc(256)
        ctr_bytes = int(N.bind("b200_gemm_allreduce_ctr_bytes", C.c_longlong, [])())
        self.off_ctr = self.heap.alloc(ctr_bytes)
        self._ctr_words = ctr_bytes // 4
        arr = self.heap.mc_array if self.use_mc else self.heap.ptr_array
        own = 0 if emulate_peers else self.rank
        if emulate_peers:
            def arr(off, _w=self.world, _h=self.heap):
                a = (C.c_void_p * _w)()
                for r in range(_w):
                    a[r] = _h.ptr(0, off)
                return a
        self._part = self.heap.ptr(own, self.off_part)
        self._part_src = arr(self.off_part)
        self._bf16 = [arr(o) for o in self.off_bf16]
        self._q = [arr(o) for o in self.off_q]
        self._sf = [arr(o) for o in self.off_sf]
        self._part_large = self.heap.ptr(own, self.off_part_large) if large_bytes else None
        self._part_large_src = arr(self.off_part_large) if large_bytes else None
        self._out_large = [arr(o) for o in self.off_out_large]
        self._next_large = 0
        self._flags = arr(self.off_flags)
        self._flags_local = self.heap.ptr(own, self.off_flags)
        self._ctr = self.heap.ptr(own, self.off_ctr)
        self._next = 0
        vp, i32, i64, f32 = C.c_void_p, C.c_int, C.c_longlong, C.c_float
        self._fn = N.bind("b200_gemm_allreduce", i32,
                          [vp, vp, i32, i32, i32, i64, i64, i32, vp, vp, vp, vp, vp, f32, i32, vp, vp, vp, vp, vp,
                           i32, vp, vp, vp, i32, i32, i32, i32, i64, i32, vp, vp, vp, vp])
        self.budget_cycles = int(config.get("wait_budget_ms")) * 2_000_000
        self.debug_skip_ready = False    # tests: withhold this rank's "ready" signal once per call

    def supports_large(self, m: int, n: int) -> bool:
        return MAX_TOKENS < m <= self.max_large_tokens and n <= self.max_features and n % 128 == 0

    def owned_rows(self, m: int) -> tuple[int, int]:
        """The block of ``m`` token rows this rank owns in the reduce-scatter / all-gather forms."""
        per = (m + self.world - 1) // self.world
        a = min(m, self.rank * per)
        return a, min(m, a + per)

    def large(self, x, w: LinearWeight, *, res: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
              slot: Optional[int] = None, scatter_out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Row-parallel linear over more than 128 tokens fused with its all-reduce and the gated
        residual add: returns ``res + gate * (sum over ranks of x_r w_r^T + bias)`` ([m, n] bf16) on
        every rank, a view of output buffer ``slot`` (one of LARGE_SLOTS; default: they take turns).
        The view is valid until a later call names the same slot; ``res`` may be the view returned by
        an earlier call with a different slot. ``res`` ([m, n] bf16, the replicated residual stream)
        and ``gate`` ([n] bf16) are optional.

        Reduce-scatter form (``scatter_out`` given: a local [owned rows, n] bf16 tensor, see
        :meth:`owned_rows`): only this rank's block of the result is produced, into ``scatter_out``
        (which is returned), and ``res`` is the rank's block of the residual stream."""
        if w.is_fp8 and not isinstance(x, Fp8Act):
            x = ops.quant_fp8_act(x, mx=w.is_mx)
        xd = x.data if isinstance(x, Fp8Act) else x
        m, k = xd.shape
        n = w.weight.shape[0]
        assert self.supports_large(m, n), (m, n, self.max_large_tokens)
        rows = m
        if scatter_out is not None:
            a, b = self.owned_rows(m)
            rows = b - a
            assert scatter_out.is_contiguous() and scatter_out.shape == (rows, n) and scatter_out.dtype == torch.bfloat16
        assert res is None or (res.is_contiguous() and res.shape == (rows, n) and res.dtype == torch.bfloat16)
        assert gate is None or (gate.is_contiguous() and gate.numel() == n and gate.dtype == torch.bfloat16)
        if slot is None:
            slot = self._next_large
            self._next_large = (self._next_large + 1) % LARGE_SLOTS
        fp8 = w.is_fp8
        st = N.state(self.device)
        rc = self._fn(xd.data_ptr(), w.weight.data_ptr(), m, n, k, xd.stride(0), w.weight.stride(0),
                      2 if w.is_mx else 1 if fp8 else 0,
                      None if not fp8 else x.sf.data_ptr() if w.is_mx else x.scale.data_ptr(),
                      None if not fp8 else w.sf.data_ptr() if w.is_mx else w.scale.data_ptr(),
                      N.ptr(w.bias), N.ptr(res), None, 0.0, 0,
                      self._part_large, self._part_large_src, self._out_large[slot], None, None, 0,
                      self._flags, self._flags_local, self._ctr, self.rank, self.world, 1 if self.use_mc else 0, 1,
                      self.budget_cycles, 0, N.ptr(gate), N.ptr(scatter_out), st.status.data_ptr(), N.stream())
        N.check(rc, "b200_gemm_allreduce")
        if scatter_out is not None:
            return scatter_out
        return self.heap.tensor(self.off_out_large[slot], (m, n), torch.bfloat16)

    def reset(self) -> None:
        """Clear the counters on every rank (all ranks call this together, with no call in
        flight). Needed after a wait that ran out: the cumulative counters no longer agree."""
        torch.cuda.synchronize(self.device)
        self.comm.barrier()
        self.heap.tensor(self.off_flags, (64,), torch.int32).zero_()
        self.heap.tensor(self.off_ctr, (self._ctr_words,), torch.int32).zero_()
        torch.cuda.synchronize(self.device)
        self.comm.barrier()

    def supports(self, m: int, n: int) -> bool:
        return 0 < m <= MAX_TOKENS and n <= self.max_features and n % 128 == 0

    def __call__(self, x, w: LinearWeight, *, res: Optional[torch.Tensor] = None,
                 norm_w: Optional[torch.Tensor] = None, eps: float = 1e-6, weight_plus_one: bool = False,
                 emit_bf16: bool = True, emit_fp8: bool = False):
        """All ranks call this together. ``res`` ([m, n] bf16, contiguous) is this rank's residual
        stream: the rows the rank owns (a contiguous block of ceil(m / world)) are read and updated
        in place, the other rows are left alone. Returns ``(h, h_fp8)``: the all-reduced (+ residual,
        + RMSNorm) activations as a bf16 tensor and / or an :class:`Fp8Act`, both views of the
        heap's output buffers (valid until the buffer comes round again, ``num_out_buffers`` calls
        later)."""
        if w.is_fp8 and not isinstance(x, Fp8Act):
            x = ops.quant_fp8_act(x, mx=w.is_mx)
        xd = x.data if isinstance(x, Fp8Act) else x
        m, k = xd.shape
        n = w.weight.shape[0]
        assert self.supports(m, n), (m, n)
        assert res is None or (res.is_contiguous() and res.shape == (m, n) and res.dtype == torch.bfloat16)
        slot = self._next
        self._next = (self._next + 1) % len(self.off_bf16)
        fp8 = w.is_fp8
        mx_out = emit_fp8 and ops.fp8_mx()
        st = N.state(self.device)
        rc = self._fn(xd.data_ptr(), w.weight.data_ptr(), m, n, k, xd.stride(0), w.weight.stride(0),
                      2 if w.is_mx else 1 if fp8 else 0,
                      None if not fp8 else x.sf.data_ptr() if w.is_mx else x.scale.data_ptr(),
                      None if not fp8 else w.sf.data_ptr() if w.is_mx else w.scale.data_ptr(),
                      N.ptr(w.bias), N.ptr(res), N.ptr(norm_w), float(eps), int(weight_plus_one),
                      self._part, self._part_src, self._bf16[slot] if emit_bf16 else None,
                      self._q[slot] if emit_fp8 else None, self._sf[slot] if emit_fp8 else None,
                      128 if mx_out else 0, self._flags, self._flags_local, self._ctr,
                      self.rank, self.world, 1 if self.use_mc else 0, PART_SPLITS, self.budget_cycles,
                      1 if self.debug_skip_ready else 0, None, None, st.status.data_ptr(), N.stream())
        N.check(rc, "b200_gemm_allreduce")
        h = self.heap.tensor(self.off_bf16[slot], (m, n), torch.bfloat16) if emit_bf16 else None
        h8 = None
        if emit_fp8:
            q = self.heap.tensor(self.off_q[slot], (m, n), torch.uint8)
            if mx_out:
                h8 = Fp8Act(q, None, self.heap.tensor(self.off_sf[slot], (1, (n + 511) // 512, 128), torch.int32), 128)
            else:
                h8 = Fp8Act(q, self.heap.tensor(self.off_sf[slot], (m, n // 128), torch.float32))
        return h, h8

    def close(self) -> None:
        self.heap.close()


class FusedColumnParallel:
    """All-gather -> GEMM in one kernel (``b200_allgather_gemm``, csrc/kernels/gemm_tcgen05.cu) for the
    column-parallel linears of a sequence-parallel region: every rank passes its block of token rows
    (:meth:`owned_rows`), the kernel copies it into every rank's gather buffer (``multimem.st``) while
    the tensor core starts on the rank's own rows, and the TMA producer waits per token tile for the
    ranks that own its rows. Returns the rank's output features for ALL tokens. More than 128 tokens.

    The reference has no sequence-parallel linears; its tensor-parallel DiT path replicates the
    activations and all-reduces after every row-parallel linear
    (src/HartsyInference.Diffusion/Models/Denoisers/TensorParallelDiT.cs)."""

    def __init__(self, comm: Comm, max_tokens: int, max_k: int, device: Optional[torch.device] = None):
        self.comm, self.rank, self.world = comm, comm.rank, comm.world
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.max_tokens, self.max_k = int(max_tokens), int(max_k)
        tiles = (self.max_tokens + 127) // 128
        act_bytes = tiles * 128 * self.max_k * 2
        sf_bytes = max(tiles * 128 * ((self.max_k + 127) // 128) * 4, tiles * ((self.max_k + 511) // 512) * 512)
        self.heap = SymmetricHeap(comm, act_bytes + sf_bytes + 8192, self.device)
        self.use_mc = self.heap.has_multicast
        self.off_act = self.heap.alloc(act_bytes, align=1024)
        self.off_sf = self.heap.alloc(sf_bytes, align=1024)
        self.off_flags = self.heap.alloc(256)
        self.off_ctr = self.heap.alloc(256)
        self._sf_bytes = sf_bytes
        # exponent bytes of rows that no rank writes (the tail of the last 128-row tile) must be finite
        self.heap.tensor(self.off_sf, (sf_bytes,), torch.uint8).fill_(127)
        torch.cuda.synchronize(self.device)
        comm.barrier()
        arr = self.heap.mc_array if self.use_mc else self.heap.ptr_array
        self._act, self._sf, self._flags = arr(self.off_act), arr(self.off_sf), arr(self.off_flags)
        self._act_local = self.heap.ptr(self.rank, self.off_act)
        self._sf_local = self.heap.ptr(self.rank, self.off_sf)
        self._flags_local = self.heap.ptr(self.rank, self.off_flags)
        self._ctr = self.heap.ptr(self.rank, self.off_ctr)
        vp, i32, i64 = C.c_void_p, C.c_int, C.c_longlong
        self._fn = N.bind("b200_allgather_gemm", i32,
                          [vp, vp, vp, vp, i32, i32, i32, i64, i64, i32, vp, vp, i32, vp, vp, vp, vp, vp, vp, vp, i32, i32,
                           i32, i64, vp, vp])
        self.budget_cycles = int(config.get("wait_budget_ms")) * 2_000_000

    def owned_rows(self, m: int) -> tuple[int, int]:
        per = (m + self.world - 1) // self.world
        a = min(m, self.rank * per)
        return a, min(m, a + per)

    def supports(self, m: int, k: int) -> bool:
        return MAX_TOKENS < m <= self.max_tokens and k <= self.max_k

    def __call__(self, x_local, w: LinearWeight, m: int, act: Optional[str] = None) -> torch.Tensor:
        """``x_local``: this rank's block of the ``m`` token rows ([rows, k] bf16, or an :class:`Fp8Act`
        when ``w`` is fp8). Returns [m, n_local] bf16."""
        if w.is_fp8 and not isinstance(x_local, Fp8Act):
            x_local = ops.quant_fp8_act(x_local, mx=w.is_mx)
        xd = x_local.data if isinstance(x_local, Fp8Act) else x_local
        a, b = self.owned_rows(m)
        k = xd.shape[1]
        assert xd.shape[0] == b - a and xd.is_contiguous() and self.supports(m, k), (xd.shape, m, a, b)
        n = w.weight.shape[0]
        out = torch.empty(m, n, dtype=torch.bfloat16, device=self.device)
        fp8 = w.is_fp8
        sc = None if not fp8 else x_local.sf if w.is_mx else x_local.scale
        st = N.state(self.device)
        rc = self._fn(xd.data_ptr(), N.ptr(sc), w.weight.data_ptr(), out.data_ptr(), m, n, k, w.weight.stride(0), n,
                      2 if w.is_mx else 1 if fp8 else 0,
                      None if not fp8 else w.sf.data_ptr() if w.is_mx else w.scale.data_ptr(), N.ptr(w.bias),
                      {None: 0, "none": 0, "gelu_tanh": 1, "silu": 2}[act], self._act, self._act_local, self._sf,
                      self._sf_local, self._flags, self._flags_local, self._ctr, self.rank, self.world,
                      1 if self.use_mc else 0, self.budget_cycles, st.status.data_ptr(), N.stream())
        N.check(rc, "b200_allgather_gemm")
        return out

    def reset(self) -> None:
        torch.cuda.synchronize(self.device)
        self.comm.barrier()
        self.heap.tensor(self.off_flags, (64,), torch.int32).zero_()
        self.heap.tensor(self.off_ctr, (64,), torch.int32).zero_()
        torch.cuda.synchronize(self.device)
        self.comm.barrier()

    def close(self) -> None:
        self.heap.close()


def enable_fused_tp(model, comm: Comm, max_tokens: int = MAX_TOKENS, autotune_tokens: int = 0,
                    large_tokens: int = 0) -> bool:
    """Route the model's row-parallel linears through the fused kernel when the shapes allow it.
    With ``autotune_tokens`` > 0 three ways of running "row-parallel linear, all-reduce, residual
    add, RMSNorm, fp8 quantisation" are timed on this model's o / down projections at that token
    count (the fused kernel; GEMM + peer-memory all-reduce kernel + norm kernel; GEMM + NCCL + norm
    kernel) and the fastest is kept. ``large_tokens`` > 0 also sizes the kernel's form for more than
    128 tokens (prefill chunks), so that their row-parallel linears end in the in-kernel all-reduce
    as well. Returns True when the fused path is active."""
    if comm.world <= 1 or not config.get("fused_comm") or config.get("p2p_disable"):
        return False
    hidden = model.cfg.hidden_size
    if hidden % 128 != 0:
        log.decision("TensorParallel", f"fused all-reduce off: hidden {hidden} is not a multiple of 128")
        return False
    dense = next((l for l in model.layers if l.o is not None and l.down is not None), None)
    if dense is None:
        # no plain attention / feed-forward pair (latent attention, expert layers): the row-parallel
        # outputs go through the stand-alone all-reduce; pick the kernel or NCCL by measurement
        if autotune_tokens <= 0:
            return False
        from .custom_ar import CustomAllReduce
        car = CustomAllReduce(comm, max(max_tokens, autotune_tokens, MAX_TOKENS) * hidden, model.device)
        t_car, t_nccl = _measure_allreduce(comm, car, autotune_tokens, hidden, model.device)
        note = (f"all-reduce of {autotune_tokens} x {hidden} bf16 (tp={comm.world}, "
                f"{'multimem' if car.use_mc else 'peer loads'}): kernel {t_car * 1e3:.1f} us, NCCL {t_nccl * 1e3:.1f} us")
        if t_car < t_nccl:
            model.custom_ar = car
            model.all_reduce = lambda y: car(y)
            log.decision("TensorParallel", "peer-memory all-reduce on; " + note)
        else:
            car.close()
            log.decision("TensorParallel", "NCCL all-reduce kept; " + note)
        return False
    fused = FusedRowParallel(comm, hidden, model.device, max_large_tokens=max(0, int(large_tokens)))

    def row_parallel(x, w: LinearWeight) -> torch.Tensor:
        m = (x.data if isinstance(x, Fp8Act) else x).shape[0]
        if fused.supports(m, w.weight.shape[0]):
            return fused(x, w)[0]
        if fused.supports_large(m, w.weight.shape[0]):
            return fused.large(x, w)
        y = ops.linear(x, w)
        return comm.all_reduce(y)

    model.row_parallel_linear = row_parallel
    model.fused_rp = fused
    if autotune_tokens > 0 and model.layers:
        from .custom_ar import CustomAllReduce
        tokens = min(autotune_tokens, MAX_TOKENS)
        car = CustomAllReduce(comm, max(max_tokens, MAX_TOKENS) * hidden, model.device)
        t_fused, t_car, t_nccl = _measure_row_parallel(model, comm, fused, car, tokens)
        best = min(t_fused, t_car, t_nccl)
        how = "multimem" if fused.use_mc else "peer loads"
        note = (f"per layer at {tokens} tokens (tp={comm.world}, {how}): fused GEMM+all-reduce+norm "
                f"{t_fused * 1e3:.1f} us, GEMM + peer-memory all-reduce + norm {t_car * 1e3:.1f} us, "
                f"GEMM + NCCL + norm {t_nccl * 1e3:.1f} us")
        if best == t_fused:
            if t_car < t_nccl:      # batches beyond the fused kernel's token limit still avoid NCCL
                model.custom_ar = car
            else:
                car.close()
            log.decision("TensorParallel", "fused GEMM+all-reduce on; " + note)
            return True
        model.row_parallel_linear = None
        model.fused_rp = None
        fused.close()
        if best == t_car:
            model.custom_ar = car
            model.all_reduce = lambda y: car(y)
            log.decision("TensorParallel", "peer-memory all-reduce on; " + note)
        else:
            car.close()
            log.decision("TensorParallel", "NCCL all-reduce kept; " + note)
        return False
    log.decision("TensorParallel", f"fused GEMM+all-reduce on for <= {MAX_TOKENS} tokens (tp={comm.world})")
    return True


def _time_graph(fn, comm: Comm, dev, inner: int = 8, reps: int = 5) -> float:
    """Device ms per call of ``fn`` replayed from a CUDA graph (the way the decode step runs it)."""
    for _ in range(3):
        fn()
    comm.barrier()
    torch.cuda.synchronize(dev)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(inner):
            fn()
    graph.replay()
    comm.barrier()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize(dev)
    ms = e0.elapsed_time(e1) / (inner * reps)
    del graph
    return ms


def _measure_allreduce(comm: Comm, car, tokens: int, hidden: int, dev) -> tuple[float, float]:
    """Device time (ms, summed over ranks) of one [tokens, hidden] bf16 all-reduce: kernel, NCCL."""
    x = torch.randn(tokens, hidden, device=dev).to(torch.bfloat16)
    times = [_time_graph(lambda: car(x), comm, dev), _time_graph(lambda: comm.all_reduce(x), comm, dev)]
    t = comm.all_reduce(torch.tensor(times, device=dev, dtype=torch.float32)) / comm.world      # mean over ranks: the same decision everywhere
    return float(t[0].item()), float(t[1].item())


def disable_fused_tp(model, comm: Comm) -> None:
    """Back to GEMM + NCCL on every rank (used after a reported wait timeout)."""
    for name in ("fused_rp", "custom_ar"):
        obj = getattr(model, name, None)
        if obj is not None:
            obj.close()
            setattr(model, name, None)
    model.row_parallel_linear = None
    model.all_reduce = comm.all_reduce


def _measure_row_parallel(model, comm: Comm, fused: FusedRowParallel, car, tokens: int) -> tuple[float, float, float]:
    """Device time (ms, summed over ranks so that every rank decides alike) of one layer's two
    row-parallel linears, each followed by all-reduce + residual add + RMSNorm (+ fp8 quantisation
    when the model's linears are fp8), through the three paths."""
    lw = next((l for l in model.layers if l.o is not None and l.down is not None), None)
    if lw is None:
        return 0.0, 1.0, 1.0
    dev = model.device
    cfg = model.cfg
    xs = [torch.randn(tokens, w.in_features, device=dev).to(torch.bfloat16) * 0.1 for w in (lw.o, lw.down)]
    ws = (lw.o, lw.down)
    res = torch.zeros(tokens, cfg.hidden_size, dtype=torch.bfloat16, device=dev)
    norm_w = lw.post_norm if lw.post_norm is not None else torch.ones(cfg.hidden_size, dtype=torch.bfloat16, device=dev)
    fp8 = bool(lw.o.is_fp8)

    def run_fused():
        for x, w in zip(xs, ws):
            fused(x, w, res=res, norm_w=norm_w, eps=cfg.rms_eps, emit_bf16=not fp8, emit_fp8=fp8)

    def run_car():
        for x, w in zip(xs, ws):
            ops.linear(x, w, out=car.input(tokens, w.out_features))
            y = car.reduce(tokens, w.out_features)
            ops.norm(y, norm_w, residual=res, eps=cfg.rms_eps, emit_fp8=fp8, emit_bf16=not fp8)

    def run_nccl():
        for x, w in zip(xs, ws):
            y = comm.all_reduce(ops.linear(x, w))
            ops.norm(y, norm_w, residual=res, eps=cfg.rms_eps, emit_fp8=fp8, emit_bf16=not fp8)

    # All candidates are timed as CUDA-graph replays, the way the decode step runs them, so that
    # host launch overhead (which differs: one launch against three or four) does not decide.
    times = [_time_graph(fn, comm, dev) for fn in (run_fused, run_car, run_nccl)]
    t = torch.tensor(times, device=dev, dtype=torch.float32)
    t = comm.all_reduce(t) / comm.world          # mean over ranks: the same decision everywhere
    return float(t[0].item()), float(t[1].item()), float(t[2].item())
