"""tcgen05 GEMM vs a plain PyTorch fp32 reference of the same op (same quantised operands)."""
import pytest
import torch

from hartsyinference_b200 import ops
from hartsyinference_b200.ops import _native as N
from hartsyinference_b200.ops import reference as R

pytestmark = pytest.mark.gpu


def _rel_err(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-6)).item()


@pytest.mark.parametrize("m,n,k", [
    (128, 128, 64), (128, 256, 128), (256, 512, 512), (1024, 768, 4096),
    (300, 200, 264), (4608, 3072, 3072), (129, 130, 72),
    (1, 128, 256), (8, 512, 1024), (16, 1000, 512), (33, 256, 640), (64, 8192, 1024), (100, 384, 2048),
])
def test_gemm_bf16(m, n, k):
    torch.manual_seed(m * 7 + n * 3 + k)
    x = (torch.randn(m, k, device="cuda") * 0.5).to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda") * 0.5).to(torch.bfloat16)
    y = ops.linear(x, ops.LinearWeight(w), splits=1)
    N.check_status()
    ref = x.float() @ w.float().t()
    assert _rel_err(y, ref) < 1e-2, _rel_err(y, ref)
    assert (y.float() - ref).abs().max().item() < 0.02 * ref.abs().max().item() + 0.05


@pytest.mark.parametrize("m,n,k,splits", [(8, 512, 4096, 4), (64, 1024, 8192, 8), (16, 130, 1024, 3), (200, 256, 2048, 2)])
def test_gemm_bf16_splitk(m, n, k, splits):
    torch.manual_seed(1)
    x = (torch.randn(m, k, device="cuda") * 0.3).to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda") * 0.3).to(torch.bfloat16)
    y = ops.linear(x, ops.LinearWeight(w), splits=splits)
    N.check_status()
    ref = x.float() @ w.float().t()
    assert _rel_err(y, ref) < 1e-2


def test_gemm_auto_splits_decode_shapes():
    torch.manual_seed(2)
    for m, n, k in [(64, 1280, 8192), (64, 1024, 3584), (4, 896, 4864)]:
        x = (torch.randn(m, k, device="cuda") * 0.3).to(torch.bfloat16)
        w = (torch.randn(n, k, device="cuda") * 0.3).to(torch.bfloat16)
        y = ops.linear(x, ops.LinearWeight(w))
        N.check_status()
        assert _rel_err(y, x.float() @ w.float().t()) < 1e-2


def test_gemm_epilogue():
    torch.manual_seed(3)
    for m in (48, 384):
        n, k = 512, 256
        x = (torch.randn(m, k, device="cuda") * 0.5).to(torch.bfloat16)
        w = (torch.randn(n, k, device="cuda") * 0.2).to(torch.bfloat16)
        b = torch.randn(n, device="cuda").to(torch.bfloat16)
        g = torch.randn(n, device="cuda").to(torch.bfloat16)
        r = torch.randn(m, n, device="cuda").to(torch.bfloat16)
        for act in (None, "gelu_tanh", "silu"):
            y = ops.linear(x, ops.LinearWeight(w, None, b), act=act, gate=g, residual=r, splits=1)
            ref = R.linear(x, w, None, None, b, act, g, r, out_dtype=torch.float32)
            assert _rel_err(y, ref) < 1e-2, (m, act)
        y = ops.linear(x, ops.LinearWeight(w, None, b), act="gelu_tanh", gate=g, residual=r, splits=2)
        ref = R.linear(x, w, None, None, b, "gelu_tanh", g, r, out_dtype=torch.float32)
        assert _rel_err(y, ref) < 1e-2
    N.check_status()


@pytest.mark.parametrize("m,n,k", [
    (128, 128, 128), (256, 384, 512), (1000, 640, 1024), (4608, 3072, 3072),
    (1, 256, 256), (16, 512, 1024), (64, 1280, 8192), (40, 200, 512), (128, 1024, 2048),
])
def test_gemm_fp8_blockscaled(m, n, k, fp8_fp32_scales):
    torch.manual_seed(m + n + k)
    x = (torch.randn(m, k, device="cuda") * torch.rand(m, 1, device="cuda") * 2).to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda") * 0.1).to(torch.bfloat16)
    wq, ws = ops.quant_fp8_weight(w)
    xa = ops.quant_fp8_act(x)
    # the quantisers themselves against their references
    wq_ref, ws_ref = R.quant_fp8_weight(w.cpu())
    assert torch.allclose(ws.cpu(), ws_ref, rtol=1e-5, atol=0)
    assert (wq.cpu().view(torch.float8_e4m3fn).float() - wq_ref.view(torch.float8_e4m3fn).float()).abs().max() <= 32
    xq_ref, xs_ref = R.quant_fp8_act(x.cpu())
    assert torch.allclose(xa.scale.cpu(), xs_ref, rtol=1e-5, atol=0)
    y = ops.linear(xa, ops.LinearWeight(wq, ws), splits=1)
    N.check_status()
    ref = R.dequant_fp8_act(xa.data, xa.scale) @ R.dequant_fp8_weight(wq, ws).t()
    assert _rel_err(y, ref) < 6e-3, _rel_err(y, ref)
    # and against the unquantised product, to catch a wrong scale layout that still self-agrees
    full = x.float() @ w.float().t()
    assert _rel_err(y, full) < 0.08


def test_gemm_fp8_splitk(fp8_fp32_scales):
    torch.manual_seed(5)
    m, n, k = 64, 1024, 8192
    x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda") * 0.1).to(torch.bfloat16)
    wq, ws = ops.quant_fp8_weight(w)
    xa = ops.quant_fp8_act(x)
    y = ops.linear(xa, ops.LinearWeight(wq, ws), splits=4)
    N.check_status()
    ref = R.dequant_fp8_act(xa.data, xa.scale) @ R.dequant_fp8_weight(wq, ws).t()
    assert _rel_err(y, ref) < 6e-3


def test_gemm_deterministic():
    torch.manual_seed(6)
    x = torch.randn(64, 4096, device="cuda").to(torch.bfloat16)
    w = torch.randn(512, 4096, device="cuda").to(torch.bfloat16)
    lw = ops.LinearWeight(w)
    a = ops.linear(x, lw, splits=4)
    b = ops.linear(x, lw, splits=4)
    assert torch.equal(a, b)


@pytest.mark.parametrize("fp8", [False, True])
def test_deferred_split_sums_match_the_reduce_kernel(fp8):
    """A small-token GEMM whose tiles are all cut along K can leave the ranges to its consumer:
    GLU and the rotary / KV-write kernel then give the results of the unfused sequence."""
    from hartsyinference_b200.ops.core import SplitSum
    torch.manual_seed(5)
    m, k = 48, 2048
    # gate|up projection -> GLU (fp8 emit)
    f = 1024
    x = (torch.randn(m, k, device="cuda") * 0.5).to(torch.bfloat16)
    w = ops.LinearWeight.from_dense((torch.randn(2 * f, k, device="cuda") * 0.05).to(torch.bfloat16), fp8=fp8)
    xin = ops.quant_fp8_act(x) if fp8 else x
    d = ops.linear(xin, w, defer=True)
    assert isinstance(d, SplitSum), "this shape has fewer tiles than SMs: the GEMM must have deferred its reduction"
    y1, q1 = ops.glu(d, "silu", emit_fp8=True)
    y0, q0 = ops.glu(ops.linear(xin, w), "silu", emit_fp8=True)
    assert torch.equal(y1, y0) and torch.equal(q1.data, q0.data)
    # qkv projection -> rotary + paged KV write
    hq, hkv, dd = 4, 2, 128
    wq = ops.LinearWeight.from_dense((torch.randn((hq + 2 * hkv) * dd, k, device="cuda") * 0.05).to(torch.bfloat16), fp8=fp8)
    pos = torch.arange(m, dtype=torch.int32, device="cuda")
    slots = torch.arange(m, dtype=torch.int64, device="cuda")
    outs = []
    for defer in (True, False):
        kc = torch.zeros(4, hkv, 16, dd, device="cuda", dtype=torch.bfloat16)
        vc = torch.zeros_like(kc)
        qkv = ops.linear(xin, wq, defer=defer)
        assert isinstance(qkv, SplitSum) == defer
        q, _, _ = ops.rope_kv(qkv, pos, hq, hkv, dd, k_cache=kc, v_cache=vc, slot_mapping=slots, theta=5e5)
        outs.append((q, kc, vc))
    for a, b in zip(outs[0], outs[1]):
        assert torch.equal(a, b)
    # a large GEMM is never deferred
    big = ops.LinearWeight.from_dense((torch.randn(148 * 128, 256, device="cuda") * 0.05).to(torch.bfloat16))
    assert isinstance(ops.linear(x[:, :256].contiguous(), big, defer=True), torch.Tensor)
