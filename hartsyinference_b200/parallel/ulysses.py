"""Sequence-parallel attention with the head/sequence exchange fused into the kernels.

Under Ulysses sequence parallelism every rank holds ``s_l`` tokens of all heads going into the
attention and needs all tokens of ``heads / world`` heads. ``FusedUlyssesAttention`` does that
exchange inside the kernels around the dense attention (csrc/kernels/attention_fa.cu):

* the operand kernel (int8 SageAttention quantisation of Q and mean-free K with their scales, or
  a plain copy in bf16 mode, and the transpose of V) stores each head group straight into the
  destination rank's operand buffers in the symmetric heap with 16-byte peer stores, and adds one
  to an arrival counter per (destination, source);
* the attention kernel walks the key segments starting with its own rank's, waits (bounded) for
  each other segment only when it gets there, and stores its output rows into the buffer of the
  rank that owns those tokens;
* a one-thread kernel waits for the ``world`` output shares before the consumer (the output
  projection) runs.

When the head count does not divide by the group size the same kernels run in their
context-parallel form (``context_parallel=True``): the queries and the output rows stay on their
rank and the K / V operands of all heads are stored into every rank's buffers, which is the
exchange the reference performs (its ranks publish K / V and read everyone else's).

A third form, ``pull=True`` (bf16 only), keeps every rank's K / V segment in its own region and lets
the attention kernel's TMA producer read each key / value tile from the owner's memory as it walks the
segments: no copies of K / V at all and ``4 x tokens / world`` rows of buffers per rank, the memory
profile of ring attention without its hop-by-hop latency (every peer is one NVSwitch hop away). The
price: a tile crosses NVLink once per query-tile pair that needs it, so this form pays off only
while a rank has few query tiles per head (short local sequences); with long local sequences the
store-once forms above move far fewer bytes and are the default.

There is no all-to-all collective and no NCCL call on this path; the NCCL all-to-all form
(models/dit/wan.py) is the fallback and the measured baseline. The reference exchanges K and V
between its device threads through a host rendezvous around every attention call
(src/HartsyInference.Diffusion/Utilities/CpKvExchange.cs:48-135; called from
Models/Denoisers/DiTBlocks/WanVideoBlock.cs:193-195).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from .. import config, log
from ..ops import _native as N
from .comm import Comm
from .symm import SymmetricHeap


class FusedUlyssesAttention:
    """One instance per (sequence-parallel group, shape). All ranks construct and call it together.

    ``local_tokens`` must be the same on every rank; head dim is 128. ``context_parallel`` defaults to
    whether ``heads`` fails to divide by the group size (the head-split form moves fewer bytes and is
    used whenever it applies).
    """

    def __init__(self, comm: Comm, local_tokens: int, heads: int, device: Optional[torch.device] = None,
                 int8: Optional[bool] = None, context_parallel: Optional[bool] = None, pull: bool = False):
        self.comm = comm
        self.rank, self.world = comm.rank, comm.world
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.s_l, self.heads = int(local_tokens), int(heads)
        self.int8 = bool(config.get("sage_attention")) if int8 is None else bool(int8)
        self.pull = bool(pull)
        if self.pull:
            self.int8 = False                   # peers hold bf16 operands only
        self.context_parallel = self.pull or (heads % self.world != 0 if context_parallel is None else bool(context_parallel))
        if self.world > 8 or (heads % self.world != 0 and not self.context_parallel):
            raise ValueError(f"{heads} heads cannot be split over {self.world} ranks")
        i32, i64, vp = C.c_int, C.c_longlong, C.c_void_p
        if self.pull:
            nbytes = int(N.bind("b200_ring_region_bytes", i64, [i32, i32, i32])(self.s_l, heads, self.world))
            self._out_off = int(N.bind("b200_ring_out_offset", i64, [i32, i32, i32])(self.s_l, heads, self.world))
        else:
            form = "b200_context_parallel" if self.context_parallel else "b200_ulysses"
            nbytes = int(N.bind(f"{form}_region_bytes", i64, [i32, i32, i32, i32])(self.s_l, heads, self.world, int(self.int8)))
            self._out_off = int(N.bind(f"{form}_out_offset", i64, [i32, i32, i32, i32])(self.s_l, heads, self.world, int(self.int8)))
        if nbytes <= 0:
            raise ValueError("unsupported exchange shape")
        self._phases = 15 | (32 if self.pull else 16 if self.context_parallel else 0)
        # plain peer stores and loads only: no multicast mapping is needed (or wanted) for this heap
        self.heap = SymmetricHeap(comm, nbytes + 4096, self.device, multicast=False)
        self.base = self.heap.alloc(nbytes, align=1024)
        self.heap.tensor(self.base, (nbytes,), torch.uint8).zero_()
        torch.cuda.synchronize(self.device)
        comm.barrier()
        self._regions = (vp * 8)()
        for r in range(self.world):
            self._regions[r] = self.heap.ptr(r, self.base)
        self._fn = N.bind("b200_ulysses_attention", i32,
                          [vp, vp, vp, vp, i32, i32, i32, i32, C.c_float, i32, C.c_uint, i32, i64, vp, vp])
        self.epoch = 0
        self.budget_cycles = int(config.get("wait_budget_ms")) * 2_000_000
        self.nbytes = nbytes
        log.decision("SequenceParallel", f"attention exchange fused into the kernels: {self.world} ranks x {self.s_l} tokens, "
                                         f"{heads} heads ({'K / V read from their owners' if self.pull else 'K / V to every rank' if self.context_parallel else 'head split'}), "
                                         f"{'int8 Q K^T' if self.int8 else 'bf16'}, {nbytes / 2**20:.0f} MiB of "
                                         f"operand buffers per rank ({self.heap.transport})")

    def __call__(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: Optional[float] = None) -> torch.Tensor:
        """q, k, v: [s_l, heads, 128] bf16 (contiguous). Returns [s_l, heads * 128] bf16, a view of the
        heap's output buffer that stays valid until the next call."""
        assert q.shape == (self.s_l, self.heads, 128) and k.shape == q.shape and v.shape == q.shape, (q.shape, self.s_l, self.heads)
        assert q.dtype == torch.bfloat16 and q.is_contiguous() and k.is_contiguous() and v.is_contiguous()
        self.epoch += 1
        st = N.state(self.device)
        rc = self._fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), self._regions, self.s_l, self.heads, self.rank, self.world,
                      float(scale if scale is not None else 128 ** -0.5), int(self.int8), self.epoch, self._phases,
                      self.budget_cycles, st.status.data_ptr(), N.stream())
        N.check(rc, "b200_ulysses_attention")
        return self.heap.tensor(self.base + self._out_off, (self.s_l, self.heads * 128), torch.bfloat16)

    def reset(self) -> None:
        """After a wait that ran out the cumulative counters disagree: all ranks call this together,
        with nothing in flight, to start again from zero."""
        torch.cuda.synchronize(self.device)
        self.comm.barrier()
        self.heap.tensor(self.base, (4096,), torch.uint8).zero_()
        self.epoch = 0
        torch.cuda.synchronize(self.device)
        self.comm.barrier()

    def close(self) -> None:
        self.heap.close()
