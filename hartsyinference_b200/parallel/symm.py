"""Symmetric heap: one equally sized device allocation per rank, mapped into every rank.

``SymmetricHeap.ptr(rank, offset)`` is an address that kernels on *this* GPU can load from and
store to, whichever GPU the memory lives on. Sub-allocations are carved with a bump allocator that
every rank advances identically, so the same offset names the same logical buffer on all ranks.
The handles are exchanged over the group's control plane and opened with CUDA IPC (C side:
``csrc/kernels/symm_heap.cu``).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from .. import log
from ..exceptions import CommError
from ..ops import _native as N
from .comm import Comm


class _RawCudaBuffer:
    """Minimal ``__cuda_array_interface__`` carrier so that torch can view heap memory."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}


class SymmetricHeap:
    def __init__(self, comm: Comm, nbytes: int, device: Optional[torch.device] = None):
        self.comm = comm
        self.rank, self.world = comm.rank, comm.world
        self.nbytes = (nbytes + 255) // 256 * 256
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        L = N.lib()
        for name, res, args in (("b200_symm_alloc", C.c_int, [C.POINTER(C.c_void_p), C.c_longlong]),
                                ("b200_symm_free", C.c_int, [C.c_void_p]),
                                ("b200_symm_export", C.c_int, [C.c_void_p, C.c_void_p]),
                                ("b200_symm_import", C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
                                ("b200_symm_unmap", C.c_int, [C.c_void_p])):
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        self._L = L
        p = C.c_void_p()
        N.check(L.b200_symm_alloc(C.byref(p), self.nbytes), "b200_symm_alloc", 0)
        self.local_ptr = p.value
        self.ptrs: list[int] = [0] * self.world
        self.ptrs[self.rank] = self.local_ptr
        self._imported: list[int] = []
        if self.world > 1:
            h = C.create_string_buffer(64)
            N.check(L.b200_symm_export(self.local_ptr, h), "b200_symm_export", 0)
            handles = comm.all_gather_object(bytes(h.raw))
            for r, raw in enumerate(handles):
                if r == self.rank:
                    continue
                q = C.c_void_p()
                buf = C.create_string_buffer(raw, 64)
                rc = L.b200_symm_import(buf, C.byref(q))
                if rc != 0:
                    raise CommError(f"cannot map the heap of rank {r} (cudaIpcOpenMemHandle code {rc})")
                self.ptrs[r] = q.value
                self._imported.append(q.value)
            comm.barrier()
        self._bump = 0
        self._view = torch.as_tensor(_RawCudaBuffer(self.local_ptr, self.nbytes), device=self.device)
        log.decision("Collective", f"symmetric heap {self.nbytes >> 20} MiB mapped on {self.world} rank(s)")

    def alloc(self, nbytes: int, align: int = 256) -> int:
        """Reserve ``nbytes``; returns the offset (identical on every rank)."""
        off = (self._bump + align - 1) // align * align
        if off + nbytes > self.nbytes:
            raise CommError(f"symmetric heap exhausted ({off + nbytes} > {self.nbytes})")
        self._bump = off + nbytes
        return off

    def ptr(self, rank: int, offset: int = 0) -> int:
        return self.ptrs[rank] + offset

    def tensor(self, offset: int, shape, dtype: torch.dtype) -> torch.Tensor:
        """A torch view of the *local* part of the heap."""
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        return self._view[offset:offset + nbytes].view(dtype).view(*shape)

    def ptr_array(self, offset: int):
        """ctypes array of the ``world`` peer addresses of one sub-allocation."""
        arr = (C.c_void_p * self.world)()
        for r in range(self.world):
            arr[r] = self.ptrs[r] + offset
        return arr

    def close(self) -> None:
        for q in self._imported:
            self._L.b200_symm_unmap(q)
        self._imported = []
        if self.local_ptr:
            self._view = None
            self._L.b200_symm_free(self.local_ptr)
            self.local_ptr = 0
