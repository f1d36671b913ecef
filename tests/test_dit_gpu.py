"""DiT forward on a B200 vs the CPU oracle (same weights), bf16 and fp8 linears."""
import pytest
import torch

from hartsyinference_b200.models.dit import flux as F
from hartsyinference_b200.models.dit import wan as W
from hartsyinference_b200.ops import _native as N

pytestmark = pytest.mark.gpu


def _cos(a, b):
    return torch.nn.functional.cosine_similarity(a.float().flatten().cpu(), b.float().flatten().cpu(), dim=0).item()


def _to(obj, dev, seen=None):
    """Deep-copy a model's tensors / LinearWeights to another device."""
    import copy
    from hartsyinference_b200.ops import LinearWeight
    new = copy.copy(obj)
    for k, v in list(obj.__dict__.items()):
        new.__dict__[k] = _mv(v, dev)
    return new


def _mv(v, dev):
    from hartsyinference_b200.ops import LinearWeight
    if isinstance(v, torch.Tensor):
        return v.to(dev)
    if isinstance(v, LinearWeight):
        return LinearWeight(_mv(v.weight, dev), _mv(v.scale, dev), _mv(v.bias, dev), _mv(v.sf, dev))
    if isinstance(v, (list, tuple)):
        return type(v)(_mv(x, dev) for x in v)
    if isinstance(v, dict):
        return {k: _mv(x, dev) for k, x in v.items()}
    if hasattr(v, "__dataclass_fields__"):
        return _to(v, dev)
    return v


@pytest.mark.parametrize("fp8", [False, True])
def test_flux_gpu_matches_cpu(fp8):
    cfg = F.tiny_flux(hidden_size=256, num_heads=2, head_dim=128, context_dim=128, pooled_dim=64, axes_dim=(16, 56, 56), in_channels=64)
    g = F.FluxTransformer(cfg, "cuda", fp8=fp8, seed=4)
    c = _to(g, "cpu")
    c.device = torch.device("cpu")
    c.fp8 = False
    gen = torch.Generator().manual_seed(0)
    img = torch.randn(1, 64, 64, generator=gen); txt = torch.randn(1, 40, 128, generator=gen); pooled = torch.randn(1, 64, generator=gen)
    ii, it = F.flux_ids(8, 8, 40)
    og = g.forward(img.cuda(), txt.cuda(), torch.tensor([0.6]).cuda(), pooled.cuda(), ii.cuda(), it.cuda(), torch.tensor([3.5]).cuda())
    oc = c.forward(img, txt, torch.tensor([0.6]), pooled, ii, it, torch.tensor([3.5]))
    N.check_status()
    assert _cos(og, oc) > (0.99 if fp8 else 0.999), _cos(og, oc)


@pytest.mark.parametrize("fp8", [False, True])
def test_flux_streamed_construction_matches_resident(fp8):
    """Blocks parked in pinned host memory as they are built and streamed through two device slots give
    the resident model's output, and hold (almost) no block weights on the device."""
    cfg = F.tiny_flux(hidden_size=256, num_heads=2, head_dim=128, context_dim=128, pooled_dim=64, axes_dim=(16, 56, 56), in_channels=64)
    resident = F.FluxTransformer(cfg, "cuda", fp8=fp8, seed=4)
    streamed = F.FluxTransformer(cfg, "cuda", fp8=fp8, seed=4, stream_blocks=True)
    assert all(b is None for b in streamed.double) and all(b is None for b in streamed.single)
    gen = torch.Generator().manual_seed(0)
    img = torch.randn(1, 64, 64, generator=gen).cuda(); txt = torch.randn(1, 40, 128, generator=gen).cuda()
    pooled = torch.randn(1, 64, generator=gen).cuda()
    ii, it = F.flux_ids(8, 8, 40)
    args = (img, txt, torch.tensor([0.6]).cuda(), pooled, ii.cuda(), it.cuda(), torch.tensor([3.5]).cuda())
    a, b = resident.forward(*args), streamed.forward(*args)
    N.check_status()
    assert torch.equal(a, b)
    assert torch.equal(streamed.forward(*args), b)          # a second pass re-streams the same blocks


@pytest.mark.parametrize("fp8", [False, True])
def test_wan_gpu_matches_cpu(fp8):
    cfg = W.tiny_wan(hidden_size=256, num_heads=2, head_dim=128, ffn_size=512, text_dim=128, text_len=32, freq_dim=64)
    g = W.WanTransformer(cfg, "cuda", fp8=fp8, seed=5)
    c = _to(g, "cpu")
    c.device = torch.device("cpu")
    c.fp8 = False
    gen = torch.Generator().manual_seed(1)
    lat = torch.randn(16, 3, 8, 8, generator=gen)
    ctx = torch.randn(32, 128, generator=gen)
    og = g.forward(lat.cuda(), torch.tensor(400.0).cuda(), g.encode_text(ctx.cuda()))
    oc = c.forward(lat, torch.tensor(400.0), c.encode_text(ctx))
    N.check_status()
    assert _cos(og, oc) > (0.99 if fp8 else 0.999), _cos(og, oc)


def test_dit_qkv_kernel():
    from hartsyinference_b200 import ops
    torch.manual_seed(0)
    t, hq, d = 77, 3, 128
    qkv = torch.randn(t, 3 * hq * d + 64, device="cuda").to(torch.bfloat16)[:, : 3 * hq * d]     # padded rows
    qw = (1 + 0.1 * torch.randn(d, device="cuda")).to(torch.bfloat16)
    kw = (1 + 0.1 * torch.randn(d, device="cuda")).to(torch.bfloat16)
    ang = torch.rand(t, d // 2, device="cuda") * 6
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    q, k, v = ops.dit_qkv(qkv, hq, hq, d, q_norm_w=qw, k_norm_w=kw, cos=cos, sin=sin)
    qr, kr, vr = ops.dit_qkv(qkv.cpu(), hq, hq, d, q_norm_w=qw.cpu(), k_norm_w=kw.cpu(), cos=cos.cpu(), sin=sin.cpu())
    for a, b in ((q, qr), (k, kr), (v, vr)):
        assert torch.allclose(a.float().cpu(), b.float(), rtol=3e-2, atol=3e-2)
