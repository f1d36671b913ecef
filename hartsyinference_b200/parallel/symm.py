"""Symmetric heap: one equally sized device allocation per rank, mapped into every rank, plus
(when the NVSwitch fabric offers it) one multicast mapping of all of them.

``SymmetricHeap.ptr(rank, offset)`` is an address that kernels on *this* GPU can load from and
store to, whichever GPU the memory lives on; ``mc_ptr(offset)`` is the multicast alias of the same
offset: a ``multimem.ld_reduce`` there returns the sum over every rank's copy (reduced inside the
switch), a ``multimem.st`` / ``multimem.red`` writes / adds to every rank's copy at once.
Sub-allocations are carved with a bump allocator that every rank advances identically, so the same
offset names the same logical buffer on all ranks.

Transports, tried in this order (C side: ``csrc/kernels/symm_heap.cu``):

1. CUDA virtual memory management: ``cuMemCreate`` allocations exported as file descriptors, sent
   between the processes as ``SCM_RIGHTS`` messages over abstract unix sockets, imported and mapped
   by every peer; rank 0 creates the multicast object, every rank adds its device, binds its
   allocation and maps the object (skipped with ``B200_NVLS=0`` or when the device reports no
   multicast support).
2. CUDA IPC handles of a ``cudaMalloc`` allocation (no multicast mapping).

A rank must take its memory out of the multicast object before it exits (:meth:`close`); a process
that dies while bound can fault its peers' links. ``close`` is registered with ``atexit`` as well.
"""
from __future__ import annotations

import atexit
import ctypes as C
import os
import socket
from typing import Optional

import torch

from .. import config, log
from ..exceptions import CommError
from ..ops import _native as N
from .comm import Comm

_uid_counter = 0


class _RawCudaBuffer:
    """Minimal ``__cuda_array_interface__`` carrier so that torch can view heap memory."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}


def _bind(L):
    vp, i32, i64, u64 = C.c_void_p, C.c_int, C.c_longlong, C.c_ulonglong
    for name, res, args in (
            ("b200_symm_alloc", i32, [C.POINTER(vp), i64]), ("b200_symm_free", i32, [vp]),
            ("b200_symm_export", i32, [vp, vp]), ("b200_symm_import", i32, [vp, C.POINTER(vp)]),
            ("b200_symm_unmap", i32, [vp]), ("b200_symm_memset", i32, [vp, i32, i64, vp]),
            ("b200_vmm_caps", i32, []), ("b200_vmm_round_size", i64, [i64, i32]),
            ("b200_vmm_create", i32, [i64, C.POINTER(u64), C.POINTER(i32)]),
            ("b200_vmm_import", i32, [i32, C.POINTER(u64)]),
            ("b200_vmm_map", i32, [u64, i64, C.POINTER(vp)]), ("b200_vmm_unmap", i32, [vp, i64]),
            ("b200_vmm_release", i32, [u64]),
            ("b200_mc_create", i32, [i32, i64, C.POINTER(u64), C.POINTER(i32)]),
            ("b200_mc_add_device", i32, [u64]), ("b200_mc_bind", i32, [u64, u64, i64]),
            ("b200_mc_unbind", i32, [u64, i64])):
        fn = getattr(L, name)
        fn.restype, fn.argtypes = res, args


def exchange_fds(comm: Comm, fds: list[int], tag: str) -> list[list[int]]:
    """Every rank contributes the same number of file descriptors; returns, per rank, that rank's
    descriptors as valid descriptors of THIS process (its own are passed through). The transfer is
    an ``SCM_RIGHTS`` message over an abstract-namespace unix socket per rank."""
    world, rank = comm.world, comm.rank
    if world == 1:
        return [list(fds)]
    name = f"\0b200-symm-{os.getuid()}-{os.getpid()}-{tag}"
    srv = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    srv.bind(name)
    srv.listen(world)
    srv.settimeout(60.0)
    try:
        names = comm.all_gather_object(name)
        for r in range(world):          # connections sit in the peer's backlog until it accepts
            if r == rank:
                continue
            c = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
            c.settimeout(60.0)
            c.connect(names[r])
            socket.send_fds(c, [rank.to_bytes(4, "little")], fds)
            c.close()
        out: list[list[int]] = [[] for _ in range(world)]
        out[rank] = list(fds)
        for _ in range(world - 1):
            conn, _ = srv.accept()
            conn.settimeout(60.0)
            msg, got, _, _ = socket.recv_fds(conn, 4, len(fds))
            conn.close()
            if len(got) != len(fds):
                raise CommError("descriptor exchange: short message")
            out[int.from_bytes(msg, "little")] = list(got)
        comm.barrier()
        return out
    finally:
        srv.close()


class SymmetricHeap:
    def __init__(self, comm: Comm, nbytes: int, device: Optional[torch.device] = None,
                 multicast: Optional[bool] = None):
        global _uid_counter
        self.comm = comm
        self.rank, self.world = comm.rank, comm.world
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        L = N.lib()
        _bind(L)
        self._L = L
        self.local_ptr = 0
        self.ptrs: list[int] = [0] * self.world
        self.mc_base = 0
        self.transport = ""
        self._mem_handle = 0
        self._mc_handle = 0
        self._peer_handles: list[int] = []
        self._imported: list[int] = []
        self._closed = False
        self._bound = False
        _uid_counter += 1
        tag = str(_uid_counter)
        want_mc = config.get("nvls") if multicast is None else multicast
        with torch.cuda.device(self.device):
            caps = L.b200_vmm_caps()
            # every rank must take the same route
            all_caps = comm.all_gather_object(int(caps)) if self.world > 1 else [int(caps)]
            vmm = all(c > 0 and (c & 1) for c in all_caps) and not config.get("symm_ipc")
            mc = vmm and want_mc and self.world > 1 and all(c & 2 for c in all_caps)
            ok = False
            if vmm:
                try:
                    ok = self._init_vmm(nbytes, mc, tag)
                except CommError as e:
                    log.warn(f"[Collective] virtual-memory heap unavailable ({e}); using CUDA IPC")
                    ok = False
                if not ok:
                    self._teardown_vmm()
            if not ok:
                self._init_ipc(nbytes)
            rc = L.b200_symm_memset(self.local_ptr, 0, self.nbytes, None)
            torch.cuda.synchronize(self.device)
            if rc != 0:
                raise CommError("cannot clear the symmetric heap")
        if self.world > 1:
            comm.barrier()
        self._bump = 0
        self._view = torch.as_tensor(_RawCudaBuffer(self.local_ptr, self.nbytes), device=self.device)
        atexit.register(self.close)
        log.decision("Collective", f"symmetric heap {self.nbytes >> 20} MiB on {self.world} rank(s), "
                                   f"transport={self.transport}, multicast={'yes' if self.mc_base else 'no'}")

    # ------------------------------------------------------------------ set-up paths
    def _agree(self, ok: bool) -> bool:
        """True when the step succeeded on every rank (a collective: all ranks call it in step)."""
        if self.world == 1:
            return bool(ok)
        return all(self.comm.all_gather_object(bool(ok)))

    def _init_vmm(self, nbytes: int, mc: bool, tag: str) -> bool:
        """Every rank walks the same sequence of collective steps, whatever fails locally."""
        L = self._L
        size = L.b200_vmm_round_size(max(nbytes, 1), self.world if mc else 1)
        sizes = self.comm.all_gather_object(int(size)) if self.world > 1 else [int(size)]
        if min(sizes) <= 0:
            raise CommError(f"allocation granularity query failed ({min(sizes)})")
        size = max(sizes)
        self.nbytes = size
        h, fd = C.c_ulonglong(), C.c_int(-1)
        rc = L.b200_vmm_create(size, C.byref(h), C.byref(fd))
        if rc == 0:
            self._mem_handle = h.value
            va = C.c_void_p()
            rc = L.b200_vmm_map(self._mem_handle, size, C.byref(va))
            if rc == 0:
                self.local_ptr = va.value
                self.ptrs[self.rank] = self.local_ptr
                self.transport = "vmm"
        if not self._agree(rc == 0):
            if fd.value >= 0:
                os.close(fd.value)
            raise CommError(f"cuMemCreate / cuMemMap failed on some rank (local code {rc})")
        if self.world > 1:
            fds = exchange_fds(self.comm, [fd.value], "mem" + tag)
            rc = 0
            for r in range(self.world):
                if r == self.rank:
                    continue
                ph = C.c_ulonglong()
                rc1 = L.b200_vmm_import(fds[r][0], C.byref(ph))
                os.close(fds[r][0])
                if rc1 == 0:
                    self._peer_handles.append(ph.value)
                    q = C.c_void_p()
                    rc1 = L.b200_vmm_map(ph.value, size, C.byref(q))
                    if rc1 == 0:
                        self.ptrs[r] = q.value
                        self._imported.append(q.value)
                rc = rc or rc1
            os.close(fd.value)
            if not self._agree(rc == 0):
                raise CommError(f"cannot import / map a peer allocation (local code {rc})")
        else:
            os.close(fd.value)
        if mc:
            self._init_multicast(size, tag)
        return True

    def _init_multicast(self, size: int, tag: str) -> None:
        """Failure here only costs the multicast alias; the peer mappings stay."""
        L = self._L
        mh, mfd = C.c_ulonglong(), C.c_int(-1)
        created = 0
        if self.rank == 0:
            created = L.b200_mc_create(self.world, size, C.byref(mh), C.byref(mfd))
        if not all(rc == 0 for rc in self.comm.all_gather_object(int(created))):
            log.warn("[Collective] multicast object could not be created; multimem paths off")
            return
        fds = exchange_fds(self.comm, [mfd.value if self.rank == 0 else os.open(os.devnull, os.O_RDONLY)], "mc" + tag)
        if self.rank != 0:
            rc = L.b200_vmm_import(fds[0][0], C.byref(mh))
        else:
            rc = 0
        for r in range(self.world):
            try:
                os.close(fds[r][0])
            except OSError:
                pass
        step_ok = all(c == 0 for c in self.comm.all_gather_object(int(rc)))
        if step_ok:
            self._mc_handle = mh.value
            rc = L.b200_mc_add_device(self._mc_handle)
            step_ok = all(c == 0 for c in self.comm.all_gather_object(int(rc)))   # also the barrier before binding
        if step_ok:
            rc = L.b200_mc_bind(self._mc_handle, self._mem_handle, size)
            self._bound = rc == 0
            step_ok = all(c == 0 for c in self.comm.all_gather_object(int(rc)))
        if step_ok:
            va = C.c_void_p()
            rc = L.b200_vmm_map(self._mc_handle, size, C.byref(va))
            if rc == 0:
                self.mc_base = va.value
            step_ok = all(c == 0 for c in self.comm.all_gather_object(int(rc)))
        if not step_ok:
            log.warn("[Collective] multicast mapping failed; multimem paths off")
            self._drop_multicast()

    def _drop_multicast(self) -> None:
        L = self._L
        if self.mc_base:
            L.b200_vmm_unmap(self.mc_base, self.nbytes)
            self.mc_base = 0
        if getattr(self, "_bound", False):
            L.b200_mc_unbind(self._mc_handle, self.nbytes)
            self._bound = False
        if self._mc_handle:
            L.b200_vmm_release(self._mc_handle)
            self._mc_handle = 0

    def _teardown_vmm(self) -> None:
        L = self._L
        self._drop_multicast()
        for q in self._imported:
            L.b200_vmm_unmap(q, self.nbytes)
        self._imported = []
        for h in self._peer_handles:
            L.b200_vmm_release(h)
        self._peer_handles = []
        if self.local_ptr and self.transport == "vmm":
            L.b200_vmm_unmap(self.local_ptr, self.nbytes)
            self.local_ptr = 0
        if self._mem_handle:
            L.b200_vmm_release(self._mem_handle)
            self._mem_handle = 0
        self.ptrs = [0] * self.world
        self.transport = ""

    def _init_ipc(self, nbytes: int) -> None:
        L = self._L
        self.nbytes = (nbytes + 255) // 256 * 256
        p = C.c_void_p()
        N.check(L.b200_symm_alloc(C.byref(p), self.nbytes), "b200_symm_alloc", 0)
        self.local_ptr = p.value
        self.ptrs[self.rank] = self.local_ptr
        self.transport = "cuda-ipc"
        if self.world > 1:
            h = C.create_string_buffer(64)
            N.check(L.b200_symm_export(self.local_ptr, h), "b200_symm_export", 0)
            handles = self.comm.all_gather_object(bytes(h.raw))
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

    # ------------------------------------------------------------------ allocation / addresses
    def alloc(self, nbytes: int, align: int = 256) -> int:
        """Reserve ``nbytes``; returns the offset (identical on every rank)."""
        off = (self._bump + align - 1) // align * align
        if off + nbytes > self.nbytes:
            raise CommError(f"symmetric heap exhausted ({off + nbytes} > {self.nbytes})")
        self._bump = off + nbytes
        return off

    def ptr(self, rank: int, offset: int = 0) -> int:
        return self.ptrs[rank] + offset

    @property
    def has_multicast(self) -> bool:
        return self.mc_base != 0

    def mc_ptr(self, offset: int = 0) -> int:
        """Multicast alias of ``offset`` (0 when the heap has no multicast mapping)."""
        return self.mc_base + offset if self.mc_base else 0

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

    def mc_array(self, offset: int):
        """One-entry ctypes array holding the multicast alias of a sub-allocation (the form the
        kernels take when they run in multimem mode)."""
        arr = (C.c_void_p * 1)()
        arr[0] = self.mc_base + offset
        return arr

    # ------------------------------------------------------------------ teardown
    def close(self) -> None:
        """Local teardown, safe to call more than once and without the peers: waits for this
        device's work, takes the allocation out of the multicast object, then unmaps and frees."""
        if self._closed:
            return
        self._closed = True
        try:
            atexit.unregister(self.close)
        except Exception:
            pass
        try:
            torch.cuda.synchronize(self.device)
        except Exception:
            pass
        self._view = None
        L = self._L
        with torch.cuda.device(self.device):
            if self.transport == "vmm":
                self._teardown_vmm()
            else:
                for q in self._imported:
                    L.b200_symm_unmap(q)
                self._imported = []
                if self.local_ptr:
                    L.b200_symm_free(self.local_ptr)
        self.local_ptr = 0
