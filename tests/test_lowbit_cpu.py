"""Low-bit codecs: exactness on representable values, error bounds on random data, layouts."""
import torch

from hartsyinference_b200.assets import lowbit as L
from hartsyinference_b200.ops import reference as R


def test_e2m1_roundtrip_and_rounding():
    codes = torch.arange(16, dtype=torch.uint8)
    vals = L.e2m1_decode(codes)
    assert vals.tolist() == [0, .5, 1, 1.5, 2, 3, 4, 6, -0.0, -.5, -1, -1.5, -2, -3, -4, -6]
    back = L.e2m1_encode(vals)
    assert torch.equal(back & 7, codes & 7) and torch.equal(back[1:8], codes[1:8]) and torch.equal(back[9:], codes[9:])
    # ties go to the even code: 0.25 -> 0, 0.75 -> 1.0, 1.25 -> 1.0, 1.75 -> 2.0, 2.5 -> 2.0, 3.5 -> 4.0, 5.0 -> 4.0
    x = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0, -5.0])
    assert L.e2m1_decode(L.e2m1_encode(x)).tolist() == [0.0, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0, 6.0, -4.0]
    p = L.pack_nibbles(codes)
    assert p.tolist() == [0x10, 0x32, 0x54, 0x76, 0x98, 0xBA, 0xDC, 0xFE] and torch.equal(L.unpack_nibbles(p), codes)


def test_mx_formats():
    g = torch.Generator().manual_seed(0)
    w = torch.randn(8, 128, generator=g) * torch.logspace(-3, 2, 8)[:, None]
    p4, s4 = L.mxfp4_quantize(w)
    assert p4.shape == (8, 64) and s4.shape == (8, 4) and s4.dtype == torch.uint8
    d4 = L.mxfp4_dequantize(p4, s4)
    assert ((d4 - w).norm() / w.norm()) < 0.15
    # values already on the grid survive exactly
    grid = L.E2M1[torch.randint(0, 8, (4, 64), generator=g)] * torch.tensor([[0.25], [1.0], [8.0], [2.0 ** -10]])
    assert torch.equal(L.mxfp4_dequantize(*L.mxfp4_quantize(grid)), grid)
    q8, s8 = L.mxfp8_quantize(w)
    d8 = L.mxfp8_dequantize(q8, s8)
    assert q8.dtype == torch.float8_e4m3fn and ((d8 - w).norm() / w.norm()) < 0.04
    # the scale is the smallest power of two that keeps the block inside the element range
    blk = w.reshape(8, 4, 32).abs().amax(-1)
    sc = L.e8m0_decode(s8)
    assert (blk / sc <= 448).all() and (blk / (sc / 2) > 448).all()
    # same power-of-two rule as the fp8 GEMM's UE8M0 activations
    assert torch.equal(L.e8m0_decode(L.e8m0_from_amax(blk, 448.0)), R.pow2_scale(blk))


def test_nvfp4_and_nf4():
    g = torch.Generator().manual_seed(1)
    w = torch.randn(16, 64, generator=g) * 0.02
    p, bs, ts = L.nvfp4_quantize(w)
    assert p.shape == (16, 32) and bs.shape == (16, 4) and bs.dtype == torch.float8_e4m3fn and ts.shape == ()
    d = L.nvfp4_dequantize(p, bs, ts)
    assert ((d - w).norm() / w.norm()) < 0.12
    assert float(bs.float().max()) <= 448.0
    pk, am = L.nf4_quantize(w)
    assert pk.shape == (512,) and am.shape == (16,)
    dn = L.nf4_dequantize(pk, am, w.shape)
    assert ((dn - w).norm() / w.norm()) < 0.1
    exact = L.NF4[torch.randint(0, 16, (128,), generator=g)] * 3.0
    exact[0] = 3.0      # the block's absmax must be present for exact recovery
    exact[64] = -3.0
    assert torch.allclose(L.nf4_dequantize(*L.nf4_quantize(exact), exact.shape), exact, atol=1e-6)


def test_blocked_scale_layout_matches_the_gemm_packing():
    g = torch.Generator().manual_seed(2)
    rows, cols = 200, 6
    sc = torch.randint(0, 255, (rows, cols), generator=g, dtype=torch.uint8)
    b = L.swizzle_block_scales(sc)
    assert b.numel() == 2 * 2 * 512
    assert torch.equal(L.unswizzle_block_scales(b, rows, cols), sc)
    # spot-check the documented address rule
    for r, c in [(0, 0), (37, 1), (127, 3), (130, 5), (199, 4)]:
        tile = (r // 128) * 2 + c // 4
        off = tile * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + (c % 4)
        assert int(b[off]) == int(sc[r, c])
    # same bytes as the UE8M0 scale-factor packing the fp8 GEMM consumes
    packed = R.pack_sf(L.e8m0_decode(sc[:128, :4].clamp(1, 253)).float(), 128).view(torch.uint8).flatten()
    assert torch.equal(packed[:512], L.swizzle_block_scales(sc[:128, :4].clamp(1, 253)))


def test_quantised_checkpoints_load_as_dense(tmp_path):
    """A llama checkpoint re-stored with fp8 block-scaled, NVFP4 and NF4 linears loads and stays close."""
    import pytest
    tr = pytest.importorskip("transformers")
    from hartsyinference_b200.models.llm.loader import load_llm, save_hf_checkpoint
    from tests.test_llm_arch_parity_cpu import _BASE, _logits
    cfg = tr.LlamaConfig(**_BASE)
    torch.manual_seed(0)
    hf = tr.AutoModelForCausalLM.from_config(cfg)
    sd = {k: (v.detach() * (3.0 if v.ndim == 2 else 1.0)).to(torch.bfloat16).contiguous() for k, v in hf.state_dict().items()}
    save_hf_checkpoint(cfg.to_dict(), sd, tmp_path / "dense")
    ids = list(range(7, 30))
    ref = _logits(load_llm(tmp_path / "dense", "cpu"), ids)

    def variant(kind):
        out = {}
        for k, v in sd.items():
            if not (k.endswith("proj.weight") and v.ndim == 2):
                out[k] = v
                continue
            w = v.float()
            if kind == "fp8_block":
                o, i = w.shape
                pad = torch.zeros(-(-o // 128) * 128, -(-i // 128) * 128)
                pad[:o, :i] = w
                amax = pad.reshape(pad.shape[0] // 128, 128, pad.shape[1] // 128, 128).abs().amax((1, 3)).clamp_min(1e-12)
                inv = amax / 448.0
                q = (w / inv.repeat_interleave(128, 0)[:o].repeat_interleave(128, 1)[:, :i]).to(torch.float8_e4m3fn)
                out[k], out[k + "_scale_inv"] = q, inv
            elif kind == "nvfp4":
                p, bs, ts = L.nvfp4_quantize(w)
                out[k], out[k + "_scale"], out[k + "_scale_2"] = p, bs, ts.reshape(1)
            elif kind == "nvfp4_ct":
                p, bs, ts = L.nvfp4_quantize(w)
                stem = k[: -len(".weight")]
                out[stem + ".weight_packed"], out[stem + ".weight_scale"], out[stem + ".weight_global_scale"] = p, bs, (1.0 / ts).reshape(1)
            elif kind == "nf4":
                p, am = L.nf4_quantize(w)
                out[k], out[k + ".absmax"], out[k + ".quant_map"] = p.reshape(-1, 1), am, L.NF4.clone()
                out[k + ".shape"] = torch.tensor(list(w.shape))
        save_hf_checkpoint(cfg.to_dict(), out, tmp_path / kind)
        return _logits(load_llm(tmp_path / kind, "cpu"), ids)

    for kind, floor in (("fp8_block", 0.995), ("nvfp4", 0.93), ("nvfp4_ct", 0.93), ("nf4", 0.95)):
        got = variant(kind)
        cos = torch.nn.functional.cosine_similarity(got.flatten(), ref.flatten(), dim=0)
        assert cos > floor, f"{kind}: {cos:.4f}"
