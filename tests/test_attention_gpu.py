"""Paged decode / prefill attention and dense attention vs the fp32 oracle."""
import pytest
import torch

from hartsyinference_b200 import ops
from hartsyinference_b200.ops import reference as R

pytestmark = pytest.mark.gpu


def _pool(pages, hkv, page, d):
    k = (torch.randn(pages, hkv, page, d, device="cuda") * 0.5).to(torch.bfloat16)
    v = (torch.randn(pages, hkv, page, d, device="cuda") * 0.5).to(torch.bfloat16)
    return k, v


@pytest.mark.parametrize("d,hq,hkv,splits", [(128, 8, 1, 1), (128, 8, 1, 4), (128, 64, 8, None), (64, 14, 2, 2), (128, 4, 4, 1), (128, 32, 2, 3)])
def test_decode_paged(d, hq, hkv, splits):
    torch.manual_seed(0)
    page, b, max_pages = 16, 5, 40
    kc, vc = _pool(256, hkv, page, d)
    lens = torch.tensor([1, 17, 300, 640, 63], dtype=torch.int32, device="cuda")
    table = torch.stack([torch.randperm(256, device="cuda")[:max_pages] for _ in range(b)]).to(torch.int32)
    q = torch.randn(b, hq, d, device="cuda").to(torch.bfloat16)
    out = ops.attn_decode(q, kc, vc, table, lens, splits=splits)
    ref = ops.attn_decode(q.cpu(), kc.cpu(), vc.cpu(), table.cpu(), lens.cpu())
    assert torch.allclose(out.float().cpu(), ref.float(), rtol=2e-2, atol=2e-2), (out.float().cpu() - ref.float()).abs().max()


@pytest.mark.parametrize("mx", [True, False])
@pytest.mark.parametrize("hq,hkv,splits", [(8, 1, 4), (12, 4, 2), (8, 2, 1)])
def test_decode_emits_fp8_for_the_output_projection(hq, hkv, splits, mx):
    """The split-combine kernel quantises its output (one 1x128 group per head); with a single
    split a separate kernel does. Either way the dequantised values match the bf16 output."""
    from hartsyinference_b200 import config
    config.set_override("fp8_scales", "ue8m0" if mx else "fp32")
    try:
        torch.manual_seed(4)
        page, b, max_pages = 16, 6, 40
        kc, vc = _pool(256, hkv, page, 128)
        lens = torch.tensor([1, 17, 300, 640, 63, 129], dtype=torch.int32, device="cuda")
        table = torch.stack([torch.randperm(256, device="cuda")[:max_pages] for _ in range(b)]).to(torch.int32)
        q = torch.randn(b, hq, 128, device="cuda").to(torch.bfloat16)
        out, o8 = ops.attn_decode(q, kc, vc, table, lens, splits=splits, emit_fp8=True)
        ref = ops.attn_decode(q.cpu(), kc.cpu(), vc.cpu(), table.cpu(), lens.cpu()).float().reshape(b, -1)
        assert torch.allclose(out.float().cpu().reshape(b, -1), ref, rtol=2e-2, atol=2e-2)
        deq = R.dequant_fp8_act(o8.data, o8.scales_fp32()).cpu()
        err = (deq - ref).norm() / ref.norm()
        assert err < 5e-2, err
        only8 = ops.attn_decode(q, kc, vc, table, lens, splits=splits, emit_fp8=True, emit_bf16=False)[1]
        assert torch.equal(only8.data, o8.data)
    finally:
        config.set_override("fp8_scales", None)


def test_decode_window_softcap():
    torch.manual_seed(1)
    page, b = 16, 3
    kc, vc = _pool(64, 2, page, 128)
    lens = torch.tensor([200, 90, 33], dtype=torch.int32, device="cuda")
    table = torch.stack([torch.randperm(64, device="cuda")[:16] for _ in range(b)]).to(torch.int32)
    q = torch.randn(b, 8, 128, device="cuda").to(torch.bfloat16)
    out = ops.attn_decode(q, kc, vc, table, lens, softcap=30.0, window=64, splits=2)
    ref = ops.attn_decode(q.cpu(), kc.cpu(), vc.cpu(), table.cpu(), lens.cpu(), softcap=30.0, window=64)
    assert torch.allclose(out.float().cpu(), ref.float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("d,hq,hkv", [(128, 8, 2), (64, 14, 2)])
def test_prefill_paged_chunked(d, hq, hkv):
    torch.manual_seed(2)
    page = 16
    kc, vc = _pool(128, hkv, page, d)
    q_lens = [70, 1, 128, 33]
    kv_lens = [70, 50, 300, 33]
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device="cuda")
    table = torch.stack([torch.randperm(128, device="cuda")[:24] for _ in range(4)]).to(torch.int32)
    q = torch.randn(sum(q_lens), hq, d, device="cuda").to(torch.bfloat16)
    lens = torch.tensor(kv_lens, dtype=torch.int32, device="cuda")
    out = ops.attn_prefill_paged(q, kc, vc, table, lens, cu, max(q_lens), causal=True)
    ref = ops.attn_prefill_paged(q.cpu(), kc.cpu(), vc.cpu(), table.cpu(), lens.cpu(), cu.cpu(), max(q_lens), causal=True)
    assert torch.allclose(out.float().cpu(), ref.float(), rtol=2e-2, atol=2e-2), (out.float().cpu() - ref.float()).abs().max()


@pytest.mark.parametrize("tq,tk,hq,hkv,d,causal", [(200, 200, 4, 4, 128, False), (130, 130, 6, 2, 64, True), (64, 333, 24, 24, 128, False), (777, 777, 2, 1, 128, True)])
def test_dense_attention(tq, tk, hq, hkv, d, causal):
    torch.manual_seed(3)
    q = torch.randn(tq, hq, d, device="cuda").to(torch.bfloat16)
    k = torch.randn(tk, hkv, d, device="cuda").to(torch.bfloat16)
    v = torch.randn(tk, hkv, d, device="cuda").to(torch.bfloat16)
    out = ops.attention(q, k, v, causal=causal)
    ref = R.attention(q.cpu(), k.cpu(), v.cpu(), causal=causal)
    assert torch.allclose(out.float().cpu(), ref, rtol=2e-2, atol=2e-2), (out.float().cpu() - ref).abs().max()
