"""CFG-parallel combine fused with the Euler step (``b200_cfg_combine``, csrc/kernels/allreduce.cu).

Rank 0 of the two-rank CFG group denoises the conditional branch, rank 1 the unconditional one.
Each copies its velocity prediction into its slot of a CUDA-IPC symmetric heap; one kernel per
rank then reads the peer's slot over NVLink, applies ``v = u + g (c - u)`` and ``z += v dt`` to the
local fp32 latents. No all_gather, no separate combine / step launches.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from .. import config
from ..ops import _native as N
from .comm import Comm
from .symm import SymmetricHeap


class FusedCfgCombine:
    def __init__(self, comm: Comm, max_elems: int, device: Optional[torch.device] = None):
        if comm.world != 2:
            raise ValueError("CFG-parallel uses exactly two ranks")
        self.comm, self.rank = comm, comm.rank
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.max_elems = (max_elems + 7) // 8 * 8
        vp, i32, i64, f32 = C.c_void_p, C.c_int, C.c_longlong, C.c_float
        self._fn = N.bind("b200_cfg_combine", i32, [vp, vp, vp, vp, vp, i64, i32, f32, f32, i64, vp, vp])
        self.heap = SymmetricHeap(comm, self.max_elems * 2 + 4096, self.device)
        self.off_pred = self.heap.alloc(self.max_elems * 2)
        self.off_flags = self.heap.alloc(256)
        self.off_ctr = self.heap.alloc(256)
        self._pred = self.heap.ptr_array(self.off_pred)
        self._flags = self.heap.ptr_array(self.off_flags)
        self._epoch = self.heap.ptr(self.rank, self.off_ctr)
        self._fin = self.heap.ptr(self.rank, self.off_ctr + 64)
        self.budget_cycles = int(config.get("wait_budget_ms")) * 2_000_000

    def slot(self, n: int) -> torch.Tensor:
        """This rank's prediction buffer (bf16 [n]); fill it before :meth:`step`."""
        return self.heap.tensor(self.off_pred, (n,), torch.bfloat16)

    def step(self, z: torch.Tensor, prediction: torch.Tensor, guidance: float, dt: float) -> torch.Tensor:
        """Both ranks call this with their branch's prediction; ``z`` (fp32, contiguous) is updated
        in place to ``z + (u + g (c - u)) dt`` on both."""
        n = z.numel()
        assert z.dtype == torch.float32 and z.is_contiguous() and prediction.numel() == n and n % 8 == 0
        assert n <= self.max_elems
        self.slot(n).copy_(prediction.reshape(-1))
        rc = self._fn(self._pred, self._flags, self._epoch, self._fin, z.data_ptr(), n, self.rank, float(guidance),
                      float(dt), self.budget_cycles, N.state(self.device).status.data_ptr(), N.stream())
        N.check(rc, "b200_cfg_combine")
        return z

    def close(self) -> None:
        self.heap.close()
