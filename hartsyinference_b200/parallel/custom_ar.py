"""Latency-oriented all-reduce for decode-sized tensors (``b200_allreduce``,
csrc/kernels/allreduce.cu): one kernel over the symmetric heap, in-switch reduction and multicast
stores (``multimem``) when the heap has a multicast mapping, peer loads / stores otherwise;
device-resident call counters (CUDA-graph capturable), bounded waits.

The producer GEMM writes its partial result straight into the heap's input buffer
(:meth:`CustomAllReduce.input`), so the collective adds no copy. Larger tensors and groups without
peer access keep using NCCL.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from .. import config
from ..ops import _native as N
from .comm import Comm
from .symm import SymmetricHeap


class CustomAllReduce:
    def __init__(self, comm: Comm, max_elems: int, device: Optional[torch.device] = None, num_out_buffers: int = 2):
        self.comm = comm
        self.rank, self.world = comm.rank, comm.world
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.max_elems = max_elems
        vp, i32, i64 = C.c_void_p, C.c_int, C.c_longlong
        self._fn = N.bind("b200_allreduce", i32, [vp, vp, vp, vp, vp, vp, i64, i32, i32, i32, i64, vp, vp])
        buf = max_elems * 2
        self.heap = SymmetricHeap(comm, buf * (1 + num_out_buffers) + 8192, self.device)
        self.use_mc = self.heap.has_multicast
        self.off_in = self.heap.alloc(buf)
        self.off_out = [self.heap.alloc(buf) for _ in range(num_out_buffers)]
        self.off_flags = self.heap.alloc(256)
        self.off_ctr = self.heap.alloc(256)
        arr = self.heap.mc_array if self.use_mc else self.heap.ptr_array
        self._in = arr(self.off_in)
        self._outs = [arr(o) for o in self.off_out]
        self._flags = arr(self.off_flags)
        self._flags_local = self.heap.ptr(self.rank, self.off_flags)
        self._ctr = self.heap.ptr(self.rank, self.off_ctr)
        self._next = 0
        self.budget_cycles = int(config.get("wait_budget_ms")) * 2_000_000

    def fits(self, elems: int) -> bool:
        return 0 < elems <= self.max_elems and elems % (8 * self.world) == 0

    def input(self, m: int, n: int) -> torch.Tensor:
        """The heap buffer to produce the local partial result in ([m, n] bf16)."""
        return self.heap.tensor(self.off_in, (m, n), torch.bfloat16)

    def reduce(self, m: int, n: int, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Sum the ``input(m, n)`` buffers of all ranks (+ this rank's ``residual``). All ranks call
        this together. Returns a view of one of the heap's output buffers (valid until that buffer
        comes round again)."""
        slot = self._next
        self._next = (self._next + 1) % len(self.off_out)
        st = N.state(self.device)
        rc = self._fn(self._in, self._outs[slot], self._flags, self._flags_local, self._ctr, N.ptr(residual), m * n,
                      self.rank, self.world, 1 if self.use_mc else 0, self.budget_cycles, st.status.data_ptr(),
                      N.stream())
        N.check(rc, "b200_allreduce")
        return self.heap.tensor(self.off_out[slot], (m, n), torch.bfloat16)

    def __call__(self, t: torch.Tensor) -> torch.Tensor:
        """Drop-in all-reduce for a tensor that was not produced in the heap (one extra copy)."""
        if t.dtype != torch.bfloat16 or not self.fits(t.numel()) or t.dim() != 2:
            return self.comm.all_reduce(t)
        m, n = t.shape
        self.input(m, n).copy_(t)
        return self.reduce(m, n)

    def close(self) -> None:
        self.heap.close()
