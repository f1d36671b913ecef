"""fp8 GEMM with UE8M0 block scales applied by the tensor core (kind::mxf8f6f4.block_scale):
quantisers, scale-factor layout and products against fp32 PyTorch statements."""
import pytest
import torch

from hartsyinference_b200 import ops
from hartsyinference_b200.ops import _native as N
from hartsyinference_b200.ops import reference as R

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel(a, b):
    return (a.float().cpu() - b.float().cpu()).abs().max().item() / (b.float().abs().max().item() + 1e-9)


def test_default_mode_is_ue8m0():
    assert ops.core.fp8_mx()


@pytest.mark.parametrize("m,k,tile_rows", [(1, 128, 128), (70, 640, 128), (300, 1024, 128), (96, 512, 16), (64, 8192, 64)])
def test_act_quantiser_and_blocked_scale_layout(m, k, tile_rows):
    torch.manual_seed(m + k)
    x = (torch.randn(m, k, device=DEV) * torch.rand(m, 1, device=DEV) * 4).to(torch.bfloat16)
    xq = ops.quant_fp8_act(x, tile_rows=tile_rows)
    assert xq.scale is None and xq.sf is not None and xq.sf.dtype == torch.int32
    q_ref, s_ref = R.quant_fp8_act(x.cpu(), pow2=True)
    s_gpu = R.unpack_sf(xq.sf.cpu(), m, k // 128, tile_rows)
    assert torch.equal(s_gpu, s_ref)                       # same power of two everywhere
    assert torch.equal(xq.data.cpu(), q_ref)
    # every assigned byte of the blocked array equals the packed reference
    b = lambda t: t.contiguous().view(torch.uint8)
    ref_sf = b(R.pack_sf(s_ref, tile_rows))
    mask = b(R.pack_sf(torch.full_like(s_ref, 2.0), tile_rows)) != b(R.pack_sf(torch.full_like(s_ref, 4.0), tile_rows))
    assert torch.equal(b(xq.sf.cpu())[mask], ref_sf[mask])


def test_norm_and_glu_emit_ue8m0():
    torch.manual_seed(2)
    x = torch.randn(50, 1024, device=DEV).to(torch.bfloat16)
    w = torch.randn(1024, device=DEV).to(torch.bfloat16)
    y, _, q = ops.norm(x, w, emit_fp8=True)
    q_ref, s_ref = R.quant_fp8_act(y.cpu(), pow2=True)
    assert torch.equal(R.unpack_sf(q.sf.cpu(), 50, 8), s_ref) and torch.equal(q.data.cpu(), q_ref)
    g = torch.randn(50, 2048, device=DEV).to(torch.bfloat16)
    a, a8 = ops.glu(g, "silu", emit_fp8=True)
    q_ref, s_ref = R.quant_fp8_act(a.cpu(), pow2=True)
    assert torch.equal(R.unpack_sf(a8.sf.cpu(), 50, 8), s_ref) and torch.equal(a8.data.cpu(), q_ref)


@pytest.mark.parametrize("m,n,k", [
    (128, 128, 128), (128, 128, 512), (256, 384, 1024), (1000, 640, 1024), (4608, 3072, 3072),
    (1, 256, 256), (16, 512, 1024), (64, 1280, 8192), (40, 200, 640), (128, 1024, 2048), (200, 256, 896),
])
def test_gemm_ue8m0_matches_dequantised_product(m, n, k):
    torch.manual_seed(m + n + k)
    x = (torch.randn(m, k, device=DEV) * torch.rand(m, 1, device=DEV) * 2).to(torch.bfloat16)
    w = (torch.randn(n, k, device=DEV) * (0.02 + 0.2 * torch.rand(n, 1, device=DEV))).to(torch.bfloat16)
    lw = ops.LinearWeight.from_dense(w, fp8=True)
    assert lw.is_mx
    xa = ops.quant_fp8_act(x)
    y = ops.linear(xa, lw, splits=1)
    N.check_status()
    ref = R.dequant_fp8_act(xa.data.cpu(), xa.scales_fp32().cpu()) @ R.dequant_fp8_weight(lw.weight.cpu(), lw.scale.cpu()).t()
    assert _rel(y, ref) < 6e-3, _rel(y, ref)
    full = x.float() @ w.float().t()
    assert _rel(y, full) < 0.1


def test_gemm_ue8m0_splitk_epilogue_and_determinism():
    torch.manual_seed(5)
    m, n, k = 64, 1024, 8192
    x = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(n, k, device=DEV) * 0.1).to(torch.bfloat16)
    b = torch.randn(n, device=DEV).to(torch.bfloat16)
    r = torch.randn(m, n, device=DEV).to(torch.bfloat16)
    lw = ops.LinearWeight.from_dense(w, b, fp8=True)
    xa = ops.quant_fp8_act(x)
    ref = R.dequant_fp8_act(xa.data.cpu(), xa.scales_fp32().cpu()) @ R.dequant_fp8_weight(lw.weight.cpu(), lw.scale.cpu()).t()
    ref = torch.nn.functional.silu(ref + b.float().cpu()) + r.float().cpu()
    for splits in (1, 4, 0):
        y = ops.linear(xa, lw, act="silu", residual=r, splits=splits)
        N.check_status()
        assert _rel(y, ref) < 8e-3, (splits, _rel(y, ref))
    assert torch.equal(ops.linear(xa, lw, splits=4), ops.linear(xa, lw, splits=4))


@pytest.mark.parametrize("groups,m,n,k", [(4, 16, 256, 512), (8, 32, 128, 1024), (3, 128, 384, 1536), (32, 16, 4096, 7168)])
def test_grouped_gemm_ue8m0(groups, m, n, k):
    torch.manual_seed(groups + m)
    x = (torch.randn(groups * m, k, device=DEV) * 0.5).to(torch.bfloat16)
    w = (torch.randn(groups * n, k, device=DEV) * 0.05).to(torch.bfloat16)
    lw = ops.LinearWeight.from_dense(w, fp8=True)
    xq = ops.quant_fp8_act(x, tile_rows=m)
    y = ops.grouped_linear(xq, lw, groups)
    N.check_status()
    xr = R.dequant_fp8_act(xq.data.cpu(), xq.scales_fp32().cpu())
    wr = R.dequant_fp8_weight(lw.weight.cpu(), lw.scale.cpu())
    ref = torch.cat([xr[g * m:(g + 1) * m] @ wr[g * n:(g + 1) * n].t() for g in range(groups)])
    assert _rel(y, ref) < 0.01
