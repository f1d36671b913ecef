"""CFG-parallel combine fused with the Euler step (``b200_cfg_combine``, csrc/kernels/allreduce.cu).

Rank 0 of the two-rank CFG group denoises the conditional branch, rank 1 the unconditional one.
Each copies its velocity prediction into its slot of a symmetric heap; one kernel per rank then
reads the peer's slot over NVLink, applies ``v = u + g (c - u)`` and either ``z += v dt`` on the
local fp32 latents (Euler) or hands ``v`` to a multi-step scheduler (UniPC). No all_gather, no
separate combine / step launches.
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
        self._fn = N.bind("b200_cfg_combine", i32, [vp, vp, vp, vp, vp, i64, i32, f32, f32, i32, i32, i64, vp, vp])
        self.heap = SymmetricHeap(comm, self.max_elems * 4 + 4096, self.device, multicast=False)
        self.off_pred = self.heap.alloc(self.max_elems * 4)
        self.off_flags = self.heap.alloc(256)
        self.off_ctr = self.heap.alloc(256)
        self._pred = self.heap.ptr_array(self.off_pred)
        self._flags = self.heap.ptr_array(self.off_flags)
        self._epoch = self.heap.ptr(self.rank, self.off_ctr)
        self._fin = self.heap.ptr(self.rank, self.off_ctr + 64)
        self.budget_cycles = int(config.get("wait_budget_ms")) * 2_000_000

    def slot(self, n: int, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        """This rank's prediction buffer ([n] bf16 or fp32); :meth:`step` / :meth:`combine` fill it."""
        return self.heap.tensor(self.off_pred, (n,), dtype)

    def _run(self, z: torch.Tensor, prediction: torch.Tensor, guidance: float, dt: float, mode: int) -> torch.Tensor:
        n = z.numel()
        assert z.dtype == torch.float32 and z.is_contiguous() and prediction.numel() == n and n % 8 == 0
        assert n <= self.max_elems
        f32 = prediction.dtype == torch.float32
        self.slot(n, torch.float32 if f32 else torch.bfloat16).copy_(prediction.reshape(-1))
        rc = self._fn(self._pred, self._flags, self._epoch, self._fin, z.data_ptr(), n, self.rank, float(guidance),
                      float(dt), mode, int(f32), self.budget_cycles, N.state(self.device).status.data_ptr(), N.stream())
        N.check(rc, "b200_cfg_combine")
        return z

    def step(self, z: torch.Tensor, prediction: torch.Tensor, guidance: float, dt: float) -> torch.Tensor:
        """Both ranks call this with their branch's prediction (bf16 or fp32); ``z`` (fp32, contiguous)
        is updated in place to ``z + (u + g (c - u)) dt`` on both."""
        return self._run(z, prediction, guidance, dt, 0)

    def combine(self, prediction: torch.Tensor, guidance: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The guided prediction ``u + g (c - u)`` itself (fp32, same shape), for schedulers whose
        update is more than an Euler step (UniPC, DPM++): both ranks call this with their branch."""
        if out is None:
            out = torch.empty(prediction.shape, dtype=torch.float32, device=prediction.device)
        self._run(out.reshape(-1), prediction, guidance, 0.0, 1)
        return out

    def close(self) -> None:
        self.heap.close()
