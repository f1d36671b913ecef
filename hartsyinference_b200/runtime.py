"""ctypes bindings to ``libb200_runtime.so`` (host-side C++: paged-KV allocator, scheduler core,
safetensors / GGUF readers, tokenizer). Built on demand when a compiler is present."""
from __future__ import annotations

import ctypes as C
import threading
from pathlib import Path
from typing import Optional

from .exceptions import KvPoolExhaustedError, NativeLibraryError

_LIB = Path(__file__).resolve().parent / "lib" / "libb200_runtime.so"
_lock = threading.Lock()
_handle: Optional[C.CDLL] = None

vp, i32, i64, u64 = C.c_void_p, C.c_int32, C.c_int64, C.c_uint64
cstr = C.c_char_p
P = C.POINTER

_SIGS = {
    "b200_kv_create": (vp, [i32, i32]),
    "b200_kv_destroy": (None, [vp]),
    "b200_kv_num_free": (i32, [vp]),
    "b200_kv_num_blocks": (i32, [vp]),
    "b200_kv_block_size": (i32, [vp]),
    "b200_kv_append": (i64, [vp, i64, i32]),
    "b200_kv_can_append": (i32, [vp, i64, i32]),
    "b200_kv_truncate": (i64, [vp, i64, i64]),
    "b200_kv_free_seq": (None, [vp, i64]),
    "b200_kv_fork_prefix": (i64, [vp, i64, i64, i64]),
    "b200_kv_seq_len": (i64, [vp, i64]),
    "b200_kv_block_table": (i32, [vp, i64, P(i32), i32]),
    "b200_kv_inject_failure": (None, [vp, i32]),
    "b200_sched_create": (vp, [vp, i32, i32, i32]),
    "b200_sched_destroy": (None, [vp]),
    "b200_sched_submit": (i32, [vp, i64, i32, i32]),
    "b200_sched_step": (i32, [vp, P(i64), P(i32), P(i32), P(i64), P(i64), i32, P(i32)]),
    "b200_sched_update": (i32, [vp, i64, i32, i32]),
    "b200_sched_abort": (i32, [vp, i64]),
    "b200_sched_stats": (None, [vp, P(i64)]),
    "b200_sched_request_state": (i32, [vp, i64, P(i32), P(i32), P(i32)]),
    "b200_st_open": (vp, [cstr]),
    "b200_st_error": (cstr, [vp]),
    "b200_st_close": (None, [vp]),
    "b200_st_count": (i32, [vp]),
    "b200_st_name": (cstr, [vp, i32]),
    "b200_st_dtype": (cstr, [vp, i32]),
    "b200_st_ndim": (i32, [vp, i32]),
    "b200_st_shape": (None, [vp, i32, P(i64)]),
    "b200_st_data": (vp, [vp, i32, P(u64)]),
    "b200_st_metadata": (cstr, [vp]),
}


def lib() -> C.CDLL:
    global _handle
    if _handle is not None:
        return _handle
    with _lock:
        if _handle is None:
            if not _LIB.exists():
                try:
                    from . import build
                    build.build_runtime()
                except Exception as e:  # pragma: no cover - depends on toolchain
                    raise NativeLibraryError(f"{_LIB} is missing and could not be built: {e}")
            h = C.CDLL(str(_LIB))
            for name, (res, args) in _SIGS.items():
                try:
                    fn = getattr(h, name)
                except AttributeError:
                    continue
                fn.restype = res
                fn.argtypes = args
            _handle = h
    return _handle


def bind(name: str, restype, argtypes):
    fn = getattr(lib(), name)
    fn.restype = restype
    fn.argtypes = argtypes
    return fn


class KvAllocator:
    """Fixed-size page pool with per-sequence block tables (C++ core)."""

    def __init__(self, num_blocks: int, block_size: int = 16):
        self._h = lib().b200_kv_create(num_blocks, block_size)
        if not self._h:
            raise ValueError("bad pool geometry")
        self.num_blocks = num_blocks
        self.block_size = block_size

    def close(self) -> None:
        if self._h:
            lib().b200_kv_destroy(self._h)
            self._h = None

    def __del__(self):  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass

    @property
    def handle(self):
        return self._h

    @property
    def num_free(self) -> int:
        return lib().b200_kv_num_free(self._h)

    def append(self, seq: int, new_tokens: int) -> int:
        r = lib().b200_kv_append(self._h, seq, new_tokens)
        if r < 0:
            raise KvPoolExhaustedError(f"no free KV page for sequence {seq} (+{new_tokens} tokens, {self.num_free} free)")
        return r

    def can_append(self, seq: int, new_tokens: int) -> bool:
        return bool(lib().b200_kv_can_append(self._h, seq, new_tokens))

    def truncate(self, seq: int, new_len: int) -> int:
        return lib().b200_kv_truncate(self._h, seq, new_len)

    def free(self, seq: int) -> None:
        lib().b200_kv_free_seq(self._h, seq)

    def fork_prefix(self, src: int, dst: int, tokens: int) -> int:
        return lib().b200_kv_fork_prefix(self._h, src, dst, tokens)

    def seq_len(self, seq: int) -> int:
        return lib().b200_kv_seq_len(self._h, seq)

    def block_table(self, seq: int, cap: int) -> list[int]:
        buf = (i32 * cap)()
        n = lib().b200_kv_block_table(self._h, seq, buf, cap)
        if n < 0:
            raise KeyError(seq)
        return list(buf[: min(n, cap)])

    def block_table_into(self, seq: int, out_ptr: int, cap: int) -> int:
        """Write the table straight into a (pinned) int32 buffer; returns the block count."""
        return lib().b200_kv_block_table(self._h, seq, C.cast(out_ptr, P(i32)), cap)

    def inject_failure(self, after_blocks: int) -> None:
        lib().b200_kv_inject_failure(self._h, after_blocks)


class SchedulerCore:
    """Continuous-batching decisions (C++ core): admission, chunked prefill, decode, pre-emption."""

    def __init__(self, kv: KvAllocator, max_batch: int = 256, prefill_token_budget: int = 8192,
                 max_prefill_seqs: int = 0, cap: int = 1024):
        self.kv = kv
        self._h = lib().b200_sched_create(kv.handle, max_batch, prefill_token_budget, max_prefill_seqs)
        self._cap = cap
        self._pid = (i64 * cap)()
        self._pst = (i32 * cap)()
        self._pct = (i32 * cap)()
        self._did = (i64 * cap)()
        self._xid = (i64 * cap)()
        self._cnt = (i32 * 3)()

    def close(self) -> None:
        if self._h:
            lib().b200_sched_destroy(self._h)
            self._h = None

    def submit(self, req_id: int, prompt_len: int, max_new_tokens: int) -> None:
        rc = lib().b200_sched_submit(self._h, req_id, prompt_len, max_new_tokens)
        if rc == -2:
            raise KvPoolExhaustedError(f"request {req_id} ({prompt_len}+{max_new_tokens} tokens) exceeds the KV pool")
        if rc != 0:
            raise ValueError(f"cannot submit request {req_id}")

    def step(self):
        """Returns (prefill [(id, start, count)], decode [id], preempted [id])."""
        lib().b200_sched_step(self._h, self._pid, self._pst, self._pct, self._did, self._xid, self._cap, self._cnt)
        np_, nd, nx = self._cnt[0], self._cnt[1], self._cnt[2]
        prefill = [(self._pid[i], self._pst[i], self._pct[i]) for i in range(np_)]
        return prefill, list(self._did[:nd]), list(self._xid[:nx])

    def update(self, req_id: int, new_tokens: int, finished: bool) -> bool:
        return lib().b200_sched_update(self._h, req_id, new_tokens, int(finished)) == 1

    def abort(self, req_id: int) -> None:
        lib().b200_sched_abort(self._h, req_id)

    def stats(self) -> dict:
        buf = (i64 * 4)()
        lib().b200_sched_stats(self._h, buf)
        return {"waiting": buf[0], "running": buf[1], "free_blocks": buf[2], "preemptions": buf[3]}

    def request_state(self, req_id: int):
        c, g, p = i32(), i32(), i32()
        st = lib().b200_sched_request_state(self._h, req_id, C.byref(c), C.byref(g), C.byref(p))
        return st, c.value, g.value, p.value
