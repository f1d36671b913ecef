"""Allocation-free GEMM entry point (``b200_gemm_noalloc``, csrc/kernels/b200_noalloc.h).

Some users of the kernels library cannot allocate device memory when they need a GEMM (a serving
loop that must stay off the allocator, a host that fixed the memory budget beforehand, a plug-in
that may not disturb its host's allocator). For them the library carries its split-K scratch in
its own image. This test calls that entry point through its exported C symbol, twice in a row so
that the second call sees the scratch the first one left behind, and compares each result with
the regular entry point (``b200_gemm`` via ``ops.linear``), which gets its scratch from the caller.
The file name sorts last on purpose: it runs after every other test, and it also passes alone in a
fresh process (the first call performs the per-device set-up).
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _entry():
    from hartsyinference_b200.ops import _native as N
    lib = C.CDLL(str(N.lib_path()))
    fn = lib.b200_gemm_noalloc
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_longlong, C.c_longlong,
                   C.c_longlong, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    return fn


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-6)).item()


@pytest.mark.parametrize("fp8", [False, True])
def test_noalloc_gemm_matches_regular_entry_twice(fp8):
    from hartsyinference_b200 import ops
    fn = _entry()
    torch.manual_seed(11)
    stream = torch.cuda.current_stream().cuda_stream
    # shapes whose tile count is not a multiple of the SM count, so the split-K scratch is used
    for m, n, k in ((64, 1280, 4096), (17, 2048, 1024)):
        x = (torch.randn(m, k, device="cuda") * 0.5).to(torch.bfloat16)
        w = (torch.randn(n, k, device="cuda") * 0.1).to(torch.bfloat16)
        bias = torch.randn(n, device="cuda").to(torch.bfloat16)
        res = torch.randn(m, n, device="cuda").to(torch.bfloat16)
        lw = ops.LinearWeight.from_dense(w, bias, fp8=fp8)
        xin = ops.quant_fp8_act(x) if fp8 else x
        ref = ops.linear(xin, lw, residual=res)
        xd = xin.data if fp8 else xin
        for call in range(2):
            out = torch.full((m, n), float("nan"), device="cuda", dtype=torch.bfloat16)
            rc = fn(xd.data_ptr(), lw.weight.data_ptr(), out.data_ptr(), m, n, k, xd.stride(0),
                    lw.weight.stride(0), out.stride(0), (2 if lw.is_mx else 1) if fp8 else 0,
                    (xin.sf if lw.is_mx else xin.scale).data_ptr() if fp8 else None,
                    (lw.sf if lw.is_mx else lw.scale).data_ptr() if fp8 else None,
                    bias.data_ptr(), res.data_ptr(), stream)
            assert rc == 0, rc
            torch.cuda.synchronize()
            assert torch.isfinite(out.float()).all()
            assert _rel(out, ref) < 1e-2, (m, n, k, call, _rel(out, ref))


def test_noalloc_gemm_with_cluster_reduction_of_the_k_splits():
    """The library-wide switch that sums K splits through distributed shared memory of a
    thread-block cluster applies to this entry point too; one small shape is checked with it on,
    then the switch goes back to what the loader had set."""
    from hartsyinference_b200 import config, ops
    from hartsyinference_b200.ops import _native as N
    fn = _entry()
    L = N.lib()
    torch.manual_seed(12)
    m, n, k = 32, 1024, 2048
    x = (torch.randn(m, k, device="cuda") * 0.5).to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda") * 0.1).to(torch.bfloat16)
    ref = ops.linear(x, ops.LinearWeight(w), splits=1)
    out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
    L.b200_gemm_set_cluster_reduce(1)
    try:
        for _ in range(2):
            rc = fn(x.data_ptr(), w.data_ptr(), out.data_ptr(), m, n, k, k, k, n, 0, None, None, None, None,
                    torch.cuda.current_stream().cuda_stream)
            assert rc == 0, rc
            torch.cuda.synchronize()
            assert _rel(out, ref) < 1e-2
    finally:
        L.b200_gemm_set_cluster_reduce(1 if config.get("cluster_splitk") else 0)


def test_noalloc_gemm_rejects_oversize():
    fn = _entry()
    x = torch.zeros(256, 256, device="cuda", dtype=torch.bfloat16)
    w = torch.zeros(256, 256, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros(256, 256, device="cuda", dtype=torch.bfloat16)
    rc = fn(x.data_ptr(), w.data_ptr(), out.data_ptr(), 256, 256, 256, 256, 256, 256, 0, None, None, None, None,
            torch.cuda.current_stream().cuda_stream)
    assert rc == -8
