"""Data-parallel attention + expert parallelism for latent-attention MoE models (DeepSeek-V2 / V3).

In the tensor-parallel layout every rank holds 1/W of the attention heads and sees all T requests of
a decode step: it reads the latent cache of ALL requests for its few heads and runs nine small
projections over all T rows. Here the requests are dealt over the ranks instead: rank r runs the
attention block of rows ``[r L, (r + 1) L)`` (L = T / W) with all heads and full (replicated)
attention weights, so per rank the cache traffic and the projection rows drop by W. The expert
layer keeps its layout (rank r owns E / W experts and computes their contribution for every row),
which needs the normalised activations of all rows on every rank before it and the sum over ranks
of the rows a rank owns after it:

    attention (L rows) -> [residual + RMSNorm -> gather to all ranks] -> router, experts, shared expert (T rows)
                       -> [combine -> scatter to the owning rank -> sum + residual + RMSNorm] -> next layer

The bracketed steps are the exchange. :class:`FusedDpExchange` does them inside the kernels that
produce and consume the data, with peer stores into a symmetric heap and cumulative arrival
counters (csrc/kernels/dp_exchange.cu); :class:`CollectiveDpExchange` states the same thing with
``all_gather`` / ``reduce_scatter`` of the communicator (CPU ranks, and the NCCL baseline the fused
form is measured against). The latent-cache row a request writes in a layer travels with the
gather, so every rank's cache stays complete: prefill chunks (which run in the tensor-parallel
layout) and any later decode step may use any rank for any request.

Reference behaviour: one device per MoE model, host routing with a device-to-host copy per layer
(src/HartsyInference.LLM/Transformer/MoeFeedForward.cs:88-161); the reference has no expert- or
data-parallel layout.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from .. import config, log, ops
from ..ops import _native as N
from .comm import Comm

LAT_ROW = 576


class CollectiveDpExchange:
    """The exchange written with the communicator's collectives (any device)."""

    fused = False

    def __init__(self, comm: Comm, max_rows: int, hidden: int, device: Optional[torch.device] = None):
        self.comm, self.rank, self.world = comm, comm.rank, comm.world
        self.max_rows, self.hidden = int(max_rows), int(hidden)
        self._partial: Optional[torch.Tensor] = None

    def supports(self, rows_total: int) -> bool:
        return rows_total % self.world == 0 and 0 < rows_total <= self.max_rows

    def gather(self, a: Optional[torch.Tensor], res: torch.Tensor, norm_w: torch.Tensor, eps: float,
               cache: Optional[torch.Tensor], slots_local: torch.Tensor, slots_all: torch.Tensor) -> torch.Tensor:
        """``res += a`` in place; returns RMSNorm(res) of ALL rows [T, H]. The cache rows written for the
        local requests in this layer are copied into the other ranks' caches on the way."""
        if a is not None:
            res.copy_((res.float() + a.float()).to(res.dtype))
        h, _, _ = ops.norm(res, norm_w, eps=eps)
        g = self.comm.all_gather(h.contiguous(), dim=0)
        if cache is not None:
            flat = cache.view(-1, LAT_ROW)
            rows = flat[slots_local.clamp(min=0).long()]
            lat = self.comm.all_gather(rows.contiguous(), dim=0)
            keep = slots_all >= 0
            flat[slots_all[keep].long()] = lat[keep]
        return g

    def scatter(self, y: Optional[torch.Tensor], slot_of: Optional[torch.Tensor], topk_w: Optional[torch.Tensor],
                shared: Optional[torch.Tensor], top_k: int) -> None:
        """This rank's contribution to every row: ``shared + sum_k w[t][k] y[slot(t, k)]``."""
        if top_k > 0:
            out = shared if shared is not None else torch.zeros(slot_of.shape[0], y.shape[1], dtype=y.dtype, device=y.device)
            ops.moe_combine(y, slot_of, topk_w, out, accumulate=shared is not None)
        else:
            out = shared
        self._partial = out

    def reduce(self, res: torch.Tensor, norm_w: torch.Tensor, eps: float) -> torch.Tensor:
        """``res += sum over ranks of the contributions to the local rows``; returns RMSNorm(res) [L, H]."""
        mine = self.comm.reduce_scatter(self._partial.contiguous(), dim=0)
        self._partial = None
        res.copy_((res.float() + mine.float()).to(res.dtype))
        h, _, _ = ops.norm(res, norm_w, eps=eps)
        return h

    def close(self) -> None:
        pass


class FusedDpExchange:
    """The exchange inside the producing / consuming kernels over a symmetric heap (CUDA ranks with
    peer access). All ranks construct and call it together."""

    fused = True

    def __init__(self, comm: Comm, max_rows: int, hidden: int, device: Optional[torch.device] = None):
        from .symm import SymmetricHeap
        self.comm, self.rank, self.world = comm, comm.rank, comm.world
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        if max_rows % self.world:
            max_rows += self.world - max_rows % self.world
        self.max_rows, self.hidden = int(max_rows), int(hidden)
        if hidden % 8 or hidden > 8192 or self.world > 8:
            raise ValueError("unsupported exchange shape")
        t, h = self.max_rows, self.hidden
        nbytes = 1024 + t * h * 2 * 2 + t * LAT_ROW * 2 + 4096
        # plain peer stores and loads only: no multicast mapping is needed for this heap
        self.heap = SymmetricHeap(comm, nbytes + 8192, self.device, multicast=False)
        self.off_flags = self.heap.alloc(256)
        self.off_ctr = self.heap.alloc(256)
        self.off_g = self.heap.alloc(t * h * 2, align=1024)
        self.off_gl = self.heap.alloc(t * LAT_ROW * 2, align=1024)
        self.off_slots = self.heap.alloc(t * h * 2, align=1024)
        self.heap.tensor(self.off_flags, (512,), torch.uint8).zero_()
        torch.cuda.synchronize(self.device)
        comm.barrier()
        self._g, self._gl = self.heap.ptr_array(self.off_g), self.heap.ptr_array(self.off_gl)
        self._slots, self._flags = self.heap.ptr_array(self.off_slots), self.heap.ptr_array(self.off_flags)
        self._flags_local = self.heap.ptr(self.rank, self.off_flags)
        self._ctr = self.heap.ptr(self.rank, self.off_ctr)
        vp, i32, i64, f32 = C.c_void_p, C.c_int, C.c_longlong, C.c_float
        self._gather = N.bind("b200_dp_norm_gather", i32, [vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, f32, vp])
        self._wait = N.bind("b200_dp_gather_wait", i32, [vp, vp, vp, vp, vp, i32, i32, i32, i64, vp, vp])
        self._scatter = N.bind("b200_dp_combine_scatter", i32, [vp, vp, vp, vp, i32, i32, vp, vp, vp, i32, i32, i32, i32, vp])
        self._reduce = N.bind("b200_dp_reduce_norm", i32, [vp, vp, vp, vp, vp, vp, i32, i32, i32, f32, i64, vp, vp])
        self.budget_cycles = int(config.get("wait_budget_ms")) * 2_000_000
        self._rows = 0
        log.decision("ExpertParallel", f"data-parallel attention exchange in the kernels: {self.world} ranks, up to "
                                       f"{self.max_rows} rows x {hidden} ({self.heap.transport})")

    def supports(self, rows_total: int) -> bool:
        return rows_total % self.world == 0 and 0 < rows_total <= self.max_rows

    def gather(self, a, res, norm_w, eps, cache, slots_local, slots_all) -> torch.Tensor:
        l = res.shape[0]
        t = l * self.world
        assert res.is_contiguous() and res.dtype == torch.bfloat16 and res.shape[1] == self.hidden and t <= self.max_rows
        assert a is None or (a.is_contiguous() and a.shape == res.shape and a.dtype == torch.bfloat16)
        assert cache is None or (cache.is_contiguous() and cache.dtype == torch.bfloat16 and cache.shape[-1] == LAT_ROW)
        assert slots_local.dtype == torch.int64 and slots_all.dtype == torch.int64 and slots_all.numel() == t
        st, stream = N.state(self.device).status.data_ptr(), N.stream()
        cp = 0 if cache is None else cache.data_ptr()
        N.check(self._gather(0 if a is None else a.data_ptr(), res.data_ptr(), norm_w.data_ptr(), cp, slots_local.data_ptr(),
                             self._g, self._gl, self._flags, self._ctr, l, self.hidden, self.rank, self.world, float(eps),
                             stream), "b200_dp_norm_gather")
        N.check(self._wait(self.heap.ptr(self.rank, self.off_gl), cp, slots_all.data_ptr(), self._flags_local, self._ctr, t, l,
                           self.rank, self.budget_cycles, st, stream), "b200_dp_gather_wait")
        self._rows = l
        return self.heap.tensor(self.off_g, (t, self.hidden), torch.bfloat16)

    def scatter(self, y, slot_of, topk_w, shared, top_k: int) -> None:
        l, t = self._rows, self._rows * self.world
        if top_k > 0:
            assert y.is_contiguous() and y.dtype == torch.bfloat16 and y.shape[1] == self.hidden
            assert slot_of.dtype == torch.int32 and topk_w.dtype == torch.float32 and slot_of.shape == (t, top_k)
        assert shared is None or (shared.is_contiguous() and shared.shape == (t, self.hidden) and shared.dtype == torch.bfloat16)
        assert top_k > 0 or shared is not None
        N.check(self._scatter(0 if top_k == 0 else y.data_ptr(), 0 if top_k == 0 else slot_of.data_ptr(),
                              0 if top_k == 0 else topk_w.data_ptr(), 0 if shared is None else shared.data_ptr(), top_k,
                              self.hidden, self._slots, self._flags, self._ctr, t, l, self.rank, self.world, N.stream()),
                "b200_dp_combine_scatter")

    def reduce(self, res, norm_w, eps) -> torch.Tensor:
        l = res.shape[0]
        h = torch.empty_like(res)
        N.check(self._reduce(self.heap.ptr(self.rank, self.off_slots), res.data_ptr(), norm_w.data_ptr(), h.data_ptr(),
                             self._flags_local, self._ctr, l, self.hidden, self.world, float(eps), self.budget_cycles,
                             N.state(self.device).status.data_ptr(), N.stream()), "b200_dp_reduce_norm")
        return h

    def reset(self) -> None:
        """After a wait that ran out the cumulative counters disagree: all ranks call this together,
        with nothing in flight, to start again from zero."""
        torch.cuda.synchronize(self.device)
        self.comm.barrier()
        self.heap.tensor(self.off_flags, (512,), torch.uint8).zero_()
        torch.cuda.synchronize(self.device)
        self.comm.barrier()

    def close(self) -> None:
        self.heap.close()


def enable_dp_attention(model, comm: Comm, max_rows: int, fused: Optional[bool] = None) -> bool:
    """Switches decode steps of ``model`` (built with ``dp_attention=True``) to the data-parallel
    attention layout. Returns whether the exchange runs in the fused kernels."""
    if comm.world <= 1 or not getattr(model, "dp_attention", False):
        return False
    dev = model.device
    want = (dev.type == "cuda" and bool(config.get("fused_dp_exchange"))) if fused is None else fused
    ex = None
    if want:
        try:
            ex = FusedDpExchange(comm, max_rows, model.cfg.hidden_size, dev)
        except Exception as e:      # no peer mapping between these GPUs: keep the collectives
            log.warn(f"[ExpertParallel] fused exchange unavailable ({type(e).__name__}: {e}); using the collectives")
    if ex is None:
        mr = max_rows + (-max_rows) % comm.world
        ex = CollectiveDpExchange(comm, mr, model.cfg.hidden_size, dev)
    model.dp_exchange = ex
    return ex.fused
