"""Fused compute + collective paths for tensor parallelism.

``FusedRowParallel`` runs the row-parallel linears of a TP group (attention output projection,
FFN down projection) as ONE kernel per linear: tcgen05 GEMM tiles whose epilogue pushes the bf16
partial tile over NVLink into the rank that owns those output columns, the owner reduces in fp32
(+ bias / residual) and pushes the result into every rank's output buffer
(``b200_gemm_allreduce``, csrc/kernels/gemm_tcgen05.cu). It covers token counts up to 128 (the
decode regime, where the all-reduce is latency-bound); larger batches use the plain GEMM and an
NCCL all-reduce, which is also the measured baseline of the fused path.

The reference performs the same two reductions per layer with ``AllReduceSum`` after the o-proj and
the down-proj (src/HartsyInference.LLM/Transformer/TensorParallelTransformer.cs:298,307) through
NCCL calls issued by one thread for all ranks (src/HartsyInference.Cuda/NcclComm.cs:53-85).
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
STAGE_SPLITS = 4      # K splits per rank that the staging buffer has slots for


class FusedRowParallel:
    def __init__(self, comm: Comm, max_features: int, device: Optional[torch.device] = None,
                 num_out_buffers: int = 2):
        self.comm = comm
        self.rank, self.world = comm.rank, comm.world
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.max_features = max_features
        tiles = (max_features + 127) // 128
        stage_bytes = STAGE_SPLITS * tiles * 128 * 128 * 2   # [world * splits][tiles/world][128][128] bf16
        out_bytes = MAX_TOKENS * max_features * 2
        flags_bytes = 4096
        self.heap = SymmetricHeap(comm, stage_bytes + num_out_buffers * out_bytes + flags_bytes + 4096, self.device)
        self.off_stage = self.heap.alloc(stage_bytes)
        self.off_out = [self.heap.alloc(out_bytes) for _ in range(num_out_buffers)]
        self.off_flags = self.heap.alloc(flags_bytes)
        # flags region: [0, 2048) tile flags (u32 each), 2048: done, 2304: epoch, 2560: fin
        self._stage = self.heap.ptr_array(self.off_stage)
        self._outs = [self.heap.ptr_array(o) for o in self.off_out]
        self._tile_flag = self.heap.ptr_array(self.off_flags)
        self._done = self.heap.ptr_array(self.off_flags + 2048)
        self._epoch = self.heap.ptr(self.rank, self.off_flags + 2304)
        self._fin = self.heap.ptr(self.rank, self.off_flags + 2560)
        self._next = 0
        vp, i32, i64, f32 = C.c_void_p, C.c_int, C.c_longlong, C.c_float
        self._fn = N.bind("b200_gemm_allreduce", i32,
                          [vp, vp, i32, i32, i32, i64, i64, i64, i32, vp, vp, vp, vp, vp, i32,
                           vp, vp, vp, vp, vp, vp, i32, i32, i32, i64, vp, vp])
        self.budget_cycles = int(config.get("wait_budget_ms")) * 2_000_000

    def supports(self, m: int, n: int) -> bool:
        return m <= MAX_TOKENS and n <= self.max_features and n % (128 * self.world) == 0

    def __call__(self, x, w: LinearWeight, residual: Optional[torch.Tensor] = None, act: Optional[str] = None,
                 gate: Optional[torch.Tensor] = None) -> torch.Tensor:
        """All ranks call this together. Returns the reduced [m, n] bf16 result, a view of one of
        the heap's output buffers (valid until the buffer comes round again)."""
        if w.is_fp8 and not isinstance(x, Fp8Act):
            x = ops.quant_fp8_act(x, mx=w.is_mx)
        xd = x.data if isinstance(x, Fp8Act) else x
        m, k = xd.shape
        n = w.weight.shape[0]
        slot = self._next
        self._next = (self._next + 1) % len(self.off_out)
        fp8 = w.is_fp8
        st = N.state(self.device)
        rc = self._fn(xd.data_ptr(), w.weight.data_ptr(), m, n, k, xd.stride(0), w.weight.stride(0), n,
                      2 if w.is_mx else 1 if fp8 else 0,
                      None if not fp8 else x.sf.data_ptr() if w.is_mx else x.scale.data_ptr(),
                      None if not fp8 else w.sf.data_ptr() if w.is_mx else w.scale.data_ptr(),
                      N.ptr(w.bias), N.ptr(gate), N.ptr(residual), {None: 0, "gelu_tanh": 1, "silu": 2}[act],
                      self._stage, self._outs[slot], self._tile_flag, self._done, self._epoch, self._fin,
                      self.rank, self.world, STAGE_SPLITS, self.budget_cycles, st.status.data_ptr(), N.stream())
        N.check(rc, "b200_gemm_allreduce")
        return self.heap.tensor(self.off_out[slot], (m, n), torch.bfloat16)

    def close(self) -> None:
        self.heap.close()


def enable_fused_tp(model, comm: Comm, max_tokens: int = MAX_TOKENS, autotune_tokens: int = 0) -> bool:
    """Route the model's row-parallel linears through the fused kernel when the shapes allow it.
    With ``autotune_tokens`` > 0 the fused kernel and GEMM + NCCL all-reduce are both timed on this
    model's o / down projections at that token count and the faster one is kept.
    Returns True when the fused path is active."""
    if comm.world <= 1 or not config.get("fused_comm") or config.get("p2p_disable"):
        return False
    hidden = model.cfg.hidden_size
    if hidden % (128 * comm.world) != 0:
        log.decision("TensorParallel", f"fused all-reduce off: hidden {hidden} not a multiple of {128 * comm.world}")
        return False
    fused = FusedRowParallel(comm, hidden, model.device)

    def row_parallel(x, w: LinearWeight) -> torch.Tensor:
        m = (x.data if isinstance(x, Fp8Act) else x).shape[0]
        if fused.supports(m, w.weight.shape[0]):
            return fused(x, w)
        y = ops.linear(x, w)
        return comm.all_reduce(y)

    model.row_parallel_linear = row_parallel
    model._fused_tp = fused
    if autotune_tokens > 0 and model.layers:
        from .custom_ar import CustomAllReduce
        car = CustomAllReduce(comm, MAX_TOKENS * hidden, model.device)
        t_fused, t_car, t_nccl = _measure_row_parallel(model, comm, fused, car, autotune_tokens)
        best = min(t_fused, t_car, t_nccl)
        note = (f"per layer at {autotune_tokens} tokens (tp={comm.world}): fused GEMM+all-reduce {t_fused * 1e3:.1f} us, "
                f"GEMM + peer-memory all-reduce {t_car * 1e3:.1f} us, GEMM + NCCL {t_nccl * 1e3:.1f} us")
        if best == t_fused:
            car.close()
            log.decision("TensorParallel", "fused GEMM+all-reduce on; " + note)
            return True
        model.row_parallel_linear = None
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


def _measure_row_parallel(model, comm: Comm, fused: FusedRowParallel, car, tokens: int) -> tuple[float, float, float]:
    """Device time (ms, summed over ranks so that every rank decides alike) of the two row-parallel
    linears of one layer through the fused kernel, through GEMM + the peer-memory all-reduce, and
    through GEMM + NCCL all-reduce."""
    lw = next((l for l in model.layers if l.o is not None and l.down is not None), None)
    if lw is None:
        return 0.0, 1.0, 1.0
    dev = model.device
    xs = [torch.randn(tokens, w.in_features, device=dev).to(torch.bfloat16) * 0.1 for w in (lw.o, lw.down)]
    ws = (lw.o, lw.down)

    def run_fused():
        for x, w in zip(xs, ws):
            fused(x, w)

    def run_car():
        for x, w in zip(xs, ws):
            ops.linear(x, w, out=car.input(tokens, w.out_features))
            car.reduce(tokens, w.out_features)

    def run_nccl():
        for x, w in zip(xs, ws):
            comm.all_reduce(ops.linear(x, w))

    # Both candidates are timed as CUDA-graph replays, the way the decode step runs them, so that
    # host launch overhead (which differs: one launch against three) does not decide.
    times = []
    inner, reps = 8, 5
    for fn in (run_fused, run_car, run_nccl):
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
        times.append(e0.elapsed_time(e1) / (inner * reps))
        del graph
    t = torch.tensor(times, device=dev, dtype=torch.float32)
    t = comm.all_reduce(t)
    return float(t[0].item()), float(t[1].item()), float(t[2].item())
