"""ctypes bindings to ``libb200_kernels.so``.

The kernels library exposes a plain C ABI (raw device pointers + ``cudaStream_t``); this module
declares the signatures, owns the per-device status word and scratch workspace, and turns
negative return codes into :class:`NativeLibraryError`. A CUDA tensor passed to an op while the
library is missing is an error, never a silent PyTorch fallback.
"""
from __future__ import annotations

import ctypes as C
import threading
from pathlib import Path
from typing import Optional

import torch

from ..exceptions import DeviceWaitTimeout, NativeLibraryError

_LIB_DIR = Path(__file__).resolve().parent.parent / "lib"
_lock = threading.Lock()
_lib: Optional[C.CDLL] = None

vp, i32, i64, f32, u64 = C.c_void_p, C.c_int, C.c_longlong, C.c_float, C.c_ulonglong

_SIGNATURES = {
    "b200_gemm": (i32, [vp, vp, vp, i32, i32, i32, i64, i64, i64, i32, vp, vp, vp, vp, vp, i32, i32, vp, i64, vp, vp]),
    "b200_gemm_workspace_bytes": (i64, []),
    "b200_gemm_set_pdl": (None, [i32]),
    "b200_gemm_set_cluster_reduce": (None, [i32]),
    "b200_gemm_set_external_reduce": (None, [i32]),
    "b200_attn_set_decode_stages": (None, [i32]),
    "b200_gemm_grouped": (i32, [vp, vp, vp, i32, i32, i32, i32, i32, vp, vp, i32, vp, i32, vp, i64, vp, vp]),
    "b200_gemm_colbatched": (i32, [vp, vp, vp, i32, i32, i32, i32, i64, i32, i64, i32, vp, i64, vp, vp]),
    "b200_mla_prep": (i32, [vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, f32, f32, vp]),
    "b200_mla_pick_splits": (i32, [i32, i32, i32]),
    "b200_mla_workspace_bytes": (i64, [i32, i32, i32]),
    "b200_mla_attn": (i32, [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, vp, f32, vp]),
    "b200_attn_fa_workspace_bytes": (i64, [i32, i32, i32, i32, i32]),
    "b200_attn_fa": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, f32, i32, vp, vp, vp]),
    "b200_attn_tc_workspace_bytes": (i64, [i32, i32, i32]),
    "b200_attn_tc": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, f32, vp, vp, vp]),
    "b200_selective_scan": (i32, [vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, vp]),
    "b200_conv_gemm": (i32, [vp, i64, i32, vp, i32, i32, vp, vp, i64, i64, vp, i32, vp, i64, vp, vp]),
    "b200_gguf_row_bytes": (i64, [i32, i32]),
    "b200_gguf_gemv_workspace_bytes": (i64, [i32, i32]),
    "b200_gguf_gemv": (i32, [vp, i64, vp, i32, vp, i64, vp, i32, i32, i32, vp, vp]),
    "b200_gguf_dequant": (i32, [vp, i32, vp, i64, i32, vp]),
    "b200_gemm_grouped_dynamic": (i32, [vp, vp, vp, i32, i32, i32, i32, i32, i32, vp, vp, i32, vp, vp, vp, vp]),
    "b200_moe_dispatch_dynamic": (i32, [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, vp]),
    "b200_moe_route": (i32, [vp, i32, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, f32, vp]),
    "b200_moe_dispatch": (i32, [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, vp]),
    "b200_moe_combine": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, vp]),
    "b200_norm": (i32, [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, f32, i32, i32, i32, vp]),
    "b200_quant_fp8": (i32, [vp, vp, vp, i32, i32, i64, i32, vp]),
    "b200_quant_fp8_weight": (i32, [vp, vp, vp, i32, i32, vp]),
    "b200_glu": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, vp, i32, i32, vp]),
    "b200_gemm_deferred": (i32, [vp, vp, vp, i32, i32, i32, i64, i64, i64, i32, vp, vp, vp, i64, vp, vp, vp]),
    "b200_rope_kv": (i32, [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, f32, f32, vp, i32, i32, vp]),
    "b200_embedding": (i32, [vp, vp, vp, i32, i32, i32, f32, vp]),
    "b200_argmax": (i32, [vp, vp, i32, i32, i64, i32, vp]),
    "b200_quant_int8_rows": (i32, [vp, vp, vp, vp, i64, i32, i64, i64, i32, vp]),
    "b200_triplane_nerf": (i32, [vp, i32, i32, i32, vp, i64, i32, C.c_float, i64, vp, vp, vp, vp, i32, vp, vp, vp, vp]),
    "b200_sample": (i32, [vp, i32, i64, i32, i32, vp, vp, vp, vp, vp, vp, vp, vp]),
    "b200_repetition_penalty": (i32, [vp, vp, vp, i32, i32, i32, vp, vp]),
    "b200_cfg_euler": (i32, [vp, vp, vp, i64, f32, f32, vp]),
    "b200_gated_residual": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, vp]),
    "b200_dit_qkv": (i32, [vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i64, f32, vp]),
    "b200_fill_random": (i32, [vp, i64, u64, f32, i32, vp]),
    "b200_attn_decode": (i32, [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, vp, f32, f32, i32, vp, vp, i32, vp]),
    "b200_attn_decode_pick_splits": (i32, [i32, i32, i32]),
    "b200_attn_decode_workspace_bytes": (i64, [i32, i32, i32, i32]),
    "b200_attn_prefill": (i32, [vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, f32, f32, vp]),
}


def lib_path() -> Path:
    """The kernels library (flag ``kernels_lib`` points at another build of it)."""
    from .. import config
    override = config.get("kernels_lib")
    return Path(override) if override else _LIB_DIR / "libb200_kernels.so"


def available() -> bool:
    return lib_path().exists()


def lib() -> C.CDLL:
    """Load (once) and return the kernels library."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            p = lib_path()
            if not p.exists():
                raise NativeLibraryError(
                    f"{p} is missing: run `python -m hartsyinference_b200.build` (needs nvcc)")
            handle = C.CDLL(str(p))
            for name, (res, args) in _SIGNATURES.items():
                try:
                    fn = getattr(handle, name)
                except AttributeError:
                    continue
                fn.restype = res
                fn.argtypes = args
            from .. import config
            try:
                handle.b200_gemm_set_pdl(1 if config.get("pdl") else 0)
                handle.b200_gemm_set_cluster_reduce(1 if config.get("cluster_splitk") else 0)
                handle.b200_gemm_set_external_reduce(1 if config.get("splitk_second_kernel") else 0)
                handle.b200_attn_set_decode_stages(int(config.get("decode_attn_stages")))
            except AttributeError:
                pass
            _lib = handle
    return _lib


def bind(name: str, restype, argtypes):
    """Declare a signature for a symbol that is not in the static table (used by sub-modules)."""
    fn = getattr(lib(), name)
    fn.restype = restype
    fn.argtypes = argtypes
    return fn


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


# number of kernels of this library launched so far by this process (ops report their own count)
launch_count = 0


def check(rc: int, what: str, launches: int = 1) -> None:
    global launch_count
    if rc != 0:
        raise NativeLibraryError(f"{what} failed with code {rc}")
    launch_count += launches


class _DeviceState:
    """Per-device status word + grow-once scratch workspace."""

    def __init__(self, device: torch.device):
        self.device = device
        self.status = torch.zeros(4, dtype=torch.int32, device=device)
        self.workspace = torch.empty(0, dtype=torch.uint8, device=device)
        self._gemm_ws = None

    def gemm_workspace(self) -> torch.Tensor:
        """Zero-initialised scratch of the GEMM's K-split path (tile counters + fp32 partials). The
        kernel leaves the counters at zero, so it is cleared here, once, and again only after a
        reported wait timeout (:meth:`reset_after_fault`)."""
        if self._gemm_ws is None:
            self._gemm_ws = torch.zeros(lib().b200_gemm_workspace_bytes(), dtype=torch.uint8, device=self.device)
        return self._gemm_ws

    def reset_after_fault(self) -> None:
        """Clear the status word and the split-K arrival counters (the first 16 KB of the GEMM
        scratch). A GEMM whose wait ran out skips its arrival, so the counters of its tiles are
        left non-zero and every later GEMM that reuses those slots would mis-detect its last
        arrival; after a reported timeout they have to be zeroed again."""
        self.status.zero_()
        if self._gemm_ws is not None:
            self._gemm_ws[:16384].zero_()

    def scratch(self, nbytes: int) -> torch.Tensor:
        if self.workspace.numel() < nbytes:
            # grow geometrically, 256-byte aligned; callers that capture CUDA graphs reserve the
            # maximum up front with reserve_workspace()
            self.workspace = torch.empty(max(nbytes, 2 * self.workspace.numel(), 1 << 20),
                                         dtype=torch.uint8, device=self.device)
        return self.workspace


_states: dict[int, _DeviceState] = {}


def state(device: torch.device) -> _DeviceState:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    st = _states.get(idx)
    if st is None:
        st = _DeviceState(torch.device("cuda", idx))
        _states[idx] = st
    return st


def reserve_workspace(device: torch.device, nbytes: int) -> None:
    state(device).scratch(nbytes)


def check_status(device: Optional[torch.device] = None, reset: bool = True) -> None:
    """Read the device status word (synchronises); raises DeviceWaitTimeout on a recorded failure."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    st = state(device)
    vals = st.status.cpu().tolist()
    if vals[0] != 0:
        if reset:
            st.reset_after_fault()
        raise DeviceWaitTimeout(
            f"device wait failed: code={vals[0]} kernel={vals[1]} site={vals[2]} detail={vals[3]}",
            kernel=vals[1], site=vals[2], detail=vals[3])
