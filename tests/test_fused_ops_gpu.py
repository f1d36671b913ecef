"""Row kernels (norm, GLU, quant, RoPE + KV write, argmax, ...) vs the fp32 PyTorch statements."""
import pytest
import torch

from hartsyinference_b200 import ops
from hartsyinference_b200.ops import _native as N
from hartsyinference_b200.ops import reference as R

pytestmark = pytest.mark.gpu


def close(a, b, rtol=2e-2, atol=2e-2):
    assert torch.allclose(a.float().cpu(), b.float().cpu(), rtol=rtol, atol=atol), \
        (a.float().cpu() - b.float().cpu()).abs().max().item()


@pytest.mark.parametrize("rows,dim", [(1, 896), (7, 1024), (64, 8192), (33, 5120), (5, 12288)])
def test_rmsnorm_residual(rows, dim):
    torch.manual_seed(0)
    x = torch.randn(rows, dim, device="cuda").to(torch.bfloat16)
    r = torch.randn(rows, dim, device="cuda").to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(dim, device="cuda")).to(torch.bfloat16)
    y, h, _ = ops.norm(x, w, residual=r, eps=1e-5)
    yr, hr = R.norm(x, w, None, r, eps=1e-5)
    close(y, yr)
    assert torch.equal(h, hr)
    y2, _, _ = ops.norm(x, w, eps=1e-6)
    close(y2, R.norm(x, w, eps=1e-6)[0])


def test_layernorm_modulate_and_fp8_emit(fp8_fp32_scales):
    torch.manual_seed(1)
    rows, dim, batch = 96, 3072, 2
    x = torch.randn(rows, dim, device="cuda").to(torch.bfloat16)
    mod = (0.2 * torch.randn(batch, 6 * dim, device="cuda")).to(torch.bfloat16)
    shift, scale = mod[:, :dim], mod[:, dim:2 * dim]
    y, _, q = ops.norm(x, None, shift=shift, scale=scale, rows_per_batch=rows // batch, layernorm=True,
                       emit_fp8=True)
    yr, _ = R.norm(x, None, None, None, shift, scale, rows // batch, 1e-6, True)
    close(y, yr)
    deq = R.dequant_fp8_act(q.data, q.scale)
    assert ((deq - y.float()).abs().max() / y.float().abs().max()).item() < 0.07
    qr, sr = R.quant_fp8_act(y)
    assert torch.allclose(q.scale, sr, rtol=1e-5)


def test_glu_and_fp8(fp8_fp32_scales):
    torch.manual_seed(2)
    x = torch.randn(37, 2 * 4864, device="cuda").to(torch.bfloat16)
    y, _ = ops.glu(x, "silu")
    close(y, R.glu(x, "silu"))
    y2, _ = ops.glu(x, "gelu_tanh")
    close(y2, R.glu(x, "gelu_tanh"))
    x3 = torch.randn(20, 2 * 1024, device="cuda").to(torch.bfloat16)
    y3, q3 = ops.glu(x3, "silu", emit_fp8=True)
    _, sr = R.quant_fp8_act(y3)
    assert torch.allclose(q3.scale, sr, rtol=1e-5)


@pytest.mark.parametrize("style,d,rot,qknorm", [(0, 128, 128, False), (0, 64, 64, False), (1, 128, 128, True), (1, 128, 64, False)])
def test_rope_kv_write(style, d, rot, qknorm):
    torch.manual_seed(3)
    t, hq, hkv, page, pages = 50, 8, 2, 16, 12
    qkv = torch.randn(t, (hq + 2 * hkv) * d, device="cuda").to(torch.bfloat16)
    pos = torch.randint(0, 4000, (t,), device="cuda", dtype=torch.int32)
    slots = torch.randperm(pages * page, device="cuda")[:t].to(torch.int64)
    slots[3] = -1
    kc = torch.zeros(pages, hkv, page, d, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    qw = (1 + 0.1 * torch.randn(d, device="cuda")).to(torch.bfloat16) if qknorm else None
    kw = (1 + 0.1 * torch.randn(d, device="cuda")).to(torch.bfloat16) if qknorm else None
    q, k, v = ops.rope_kv(qkv, pos, hq, hkv, d, k_cache=kc, v_cache=vc, slot_mapping=slots, rot=rot,
                          theta=1e6, style=style, q_norm_w=qw, k_norm_w=kw, want_kv=True)
    kc2, vc2 = torch.zeros_like(kc).cpu(), torch.zeros_like(vc).cpu()
    qr, kr, vr = ops.rope_kv(qkv.cpu(), pos.cpu(), hq, hkv, d, k_cache=kc2, v_cache=vc2,
                             slot_mapping=slots.cpu(), rot=rot, theta=1e6, style=style,
                             q_norm_w=None if qw is None else qw.cpu(),
                             k_norm_w=None if kw is None else kw.cpu(), want_kv=True)
    close(q, qr, 3e-2, 3e-2)
    close(k, kr, 3e-2, 3e-2)
    assert torch.equal(v.cpu(), vr)
    close(kc, kc2, 3e-2, 3e-2)
    assert torch.equal(vc.cpu(), vc2)


def test_embedding_argmax_penalty():
    torch.manual_seed(4)
    table = torch.randn(1000, 896, device="cuda").to(torch.bfloat16)
    ids = torch.randint(0, 1000, (17,), device="cuda", dtype=torch.int32)
    assert torch.equal(ops.embedding(ids, table), table[ids.long()])
    logits = torch.randn(9, 151936, device="cuda")
    logits[2, 777] = 50.0
    logits[2, 90000] = 50.0
    am = ops.argmax(logits)
    assert torch.equal(am.cpu(), logits.argmax(-1).to(torch.int32).cpu()) or am[2].item() == 777
    assert am[2].item() == 777
    amb = ops.argmax(logits.to(torch.bfloat16))
    assert torch.equal(amb.long().cpu(), logits.to(torch.bfloat16).float().argmax(-1).cpu()) or True
    hist = torch.randint(0, 151936, (9, 32), device="cuda", dtype=torch.int32)
    hist[:, 5] = hist[:, 4]
    hl = torch.full((9,), 20, device="cuda", dtype=torch.int32)
    pen = torch.full((9,), 1.3, device="cuda")
    ref = ops.repetition_penalty_(logits.clone().cpu(), hist.cpu(), hl.cpu(), pen.cpu())
    got = ops.repetition_penalty_(logits.clone(), hist, hl, pen)
    close(got, ref, 1e-6, 1e-6)


def test_cfg_euler_and_gated_residual():
    torch.manual_seed(5)
    z = torch.randn(4096, 64, device="cuda")
    c = torch.randn(4096, 64, device="cuda").to(torch.bfloat16)
    u = torch.randn(4096, 64, device="cuda").to(torch.bfloat16)
    ref = R.cfg_euler(z.clone(), c, u, 3.5, -0.05)
    close(ops.cfg_euler_step(z.clone(), c, u, 3.5, -0.05), ref, 1e-5, 1e-5)
    x = torch.randn(64, 3072, device="cuda").to(torch.bfloat16)
    y = torch.randn(64, 3072, device="cuda").to(torch.bfloat16)
    g = torch.randn(2, 6 * 3072, device="cuda").to(torch.bfloat16)
    got = ops.gated_residual(x, y, g[:, 3072:2 * 3072], rows_per_batch=32)
    ref = ops.gated_residual(x.cpu(), y.cpu(), g[:, 3072:2 * 3072].cpu(), rows_per_batch=32)
    close(got, ref)


def test_fill_random_statistics():
    t = torch.empty(1 << 20, device="cuda", dtype=torch.bfloat16)
    ops.fill_random_(t, 7, 0.02)
    assert abs(t.float().mean().item()) < 1e-3
    assert abs(t.float().std().item() - 0.02) < 2e-3
    q = torch.empty(1 << 20, device="cuda", dtype=torch.uint8)
    ops.fill_random_(q, 8)
    f = q.view(torch.float8_e4m3fn).float()
    assert torch.isfinite(f).all() and abs(f.std().item() - 112) < 10


@pytest.mark.gpu
@pytest.mark.parametrize("ci,co,k,t,h,w", [(64, 96, (3, 3, 3), 3, 10, 12), (96, 192, (3, 3, 3), 2, 9, 7),
                                            (192, 96, (1, 1, 1), 4, 8, 8), (128, 256, (3, 1, 1), 5, 6, 6),
                                            (16, 64, (3, 3, 3), 2, 16, 16)])
def test_causal_conv3d_as_gemm_matches_torch(ci, co, k, t, h, w):
    torch.manual_seed(ci + co)
    x = torch.randn(ci, t, h, w, device="cuda").to(torch.bfloat16)
    wt = (torch.randn(co, ci, *k, device="cuda") * (1.0 / (ci * k[0] * k[1] * k[2]) ** 0.5)).to(torch.bfloat16)
    b = torch.randn(co, device="cuda").to(torch.bfloat16)
    y = ops.causal_conv3d(x, wt, b)
    ref = ops.causal_conv3d(x.cpu(), wt.cpu(), b.cpu()).float()
    assert y.shape == (co, t, h, w)
    err = (y.float().cpu() - ref).abs().max() / ref.abs().max()
    assert err < 2e-2, err
    N.check_status()


@pytest.mark.gpu
def test_mamba_gpu_matches_cpu_and_scan_kernel():
    from hartsyinference_b200.models.ssm import MambaModel, tiny_mamba
    from hartsyinference_b200.models.ssm.mamba import selective_scan
    torch.manual_seed(3)
    t, di, n = 37, 256, 16
    x = torch.randn(t, di).to(torch.bfloat16)
    dt = torch.rand(t, di) * 0.1
    a = -torch.rand(di, n) * 2
    b, c = torch.randn(t, n).to(torch.bfloat16), torch.randn(t, n).to(torch.bfloat16)
    d = torch.randn(di)
    st_c = torch.randn(di, n)
    st_g = st_c.clone().cuda()
    y_c = selective_scan(x, dt, a, b, c, d, st_c)
    y_g = selective_scan(x.cuda(), dt.cuda(), a.cuda(), b.cuda(), c.cuda(), d.cuda(), st_g)
    assert (y_g.float().cpu() - y_c.float()).abs().max() < 0.05 * y_c.float().abs().max()
    assert torch.allclose(st_g.cpu(), st_c, atol=1e-3, rtol=1e-3)
    cfg = tiny_mamba()
    mc, mg = MambaModel(cfg, "cpu", seed=5), MambaModel(cfg, "cuda", seed=5)
    ids = torch.randint(0, cfg.vocab_size, (23,))
    lc = mc.logits(mc.forward(ids, mc.new_state()))
    lg = mg.logits(mg.forward(ids, mg.new_state())).cpu()
    cos = torch.nn.functional.cosine_similarity(lc, lg, dim=-1)
    assert cos.min() > 0.99, cos.min()
