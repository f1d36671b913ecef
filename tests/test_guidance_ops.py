"""Guidance normalisations and the multistep-solver update (csrc/kernels/guidance.cu) against their fp32
statements (ops/reference.py), on CPU by definition and on the device by kernel."""
import pytest
import torch

from hartsyinference_b200 import ops
from hartsyinference_b200.ops import reference as R


def test_reference_forms():
    torch.manual_seed(0)
    z, c, u = torch.randn(3, 5, 8), torch.randn(3, 5, 8), torch.randn(3, 5, 8)
    g, dt = 4.0, -0.1
    guided = u + g * (c - u)
    s = float((c.norm() / guided.norm()).clamp(0.3, 1.0))
    assert torch.allclose(R.cfg_renorm_euler(z, c, u, g, dt, 0.3), z + guided * s * dt, atol=1e-6)
    assert torch.allclose(R.cfg_renorm_euler(z, c, u, g, dt, 0.99), z + guided * 0.99 * dt, atol=1e-6)
    row = c.norm(dim=-1, keepdim=True) / guided.norm(dim=-1, keepdim=True)
    assert torch.allclose(R.cfg_rownorm_euler(z, c, u, g, dt), z + guided * row * dt, atol=1e-5)
    zero = torch.zeros(2, 4)
    assert torch.equal(R.cfg_rownorm_euler(zero.clone(), zero, zero, 3.0, 1.0, eps=0.0), zero)      # 0 / 0 rows stay 0
    out = ops.lincomb([(0.5, z), (-2.0, c), (3.0, u)])
    assert torch.allclose(out, 0.5 * z - 2.0 * c + 3.0 * u, atol=1e-6)
    z2 = z.clone()
    assert ops.cfg_renorm_euler_step(z2, c, u, g, dt, 0.3) is z2 and torch.allclose(z2, R.cfg_renorm_euler(z, c, u, g, dt, 0.3))


def test_scheduler_uses_the_normalised_steps():
    from hartsyinference_b200.models.diffusion.schedulers import FlowMatchEulerScheduler
    torch.manual_seed(1)
    s = FlowMatchEulerScheduler(4)
    z, c, u = torch.randn(1, 6, 16), torch.randn(1, 6, 16), torch.randn(1, 6, 16)
    a = s.step(z.clone(), c, 1, u, 3.0, renorm_min=0.0)
    assert torch.allclose(a, R.cfg_renorm_euler(z, c, u, 3.0, s.dt(1), 0.0), atol=1e-6)
    b = s.step(z.clone(), c, 1, u, 3.0, row_norm=True)
    assert torch.allclose(b, R.cfg_rownorm_euler(z, c, u, 3.0, s.dt(1)), atol=1e-5)
    plain = s.step(z.clone(), c, 1, u, 3.0)
    assert not torch.allclose(plain, a)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("n_rows,dim", [(1, 7), (300, 64), (4608, 3072 // 48), (37, 1000)])
def test_kernels_match_reference(dtype, n_rows, dim):
    torch.manual_seed(2)
    dev = "cuda"
    z = torch.randn(n_rows, dim, device=dev)
    c = torch.randn(n_rows, dim, device=dev).to(dtype)
    u = (torch.randn(n_rows, dim, device=dev) * 0.7).to(dtype)
    for rmin in (0.0, 0.9):
        for _ in range(2):                          # the second call reuses the scratch counters
            got = ops.cfg_renorm_euler_step(z.clone(), c, u, 5.0, -0.07, rmin)
            want = R.cfg_renorm_euler(z.cpu(), c.cpu(), u.cpu(), 5.0, -0.07, rmin)
            assert (got.cpu() - want).abs().max() < 1e-4
    got = ops.cfg_rownorm_euler_step(z.clone(), c, u, 5.0, -0.07)
    want = R.cfg_rownorm_euler(z.cpu(), c.cpu(), u.cpu(), 5.0, -0.07)
    assert (got.cpu() - want).abs().max() < 1e-4
    xs = [torch.randn(n_rows * dim, device=dev) for _ in range(4)]
    coefs = [0.3, -1.5, 2.0, 0.01]
    out = ops.lincomb(list(zip(coefs, xs)))
    assert (out - sum(k * x for k, x in zip(coefs, xs))).abs().max() < 1e-5
    ops.lincomb([(1.0, xs[0]), (2.0, xs[1])], out=xs[0])        # in place
    assert torch.isfinite(xs[0]).all()


@pytest.mark.gpu
def test_unipc_on_the_device_matches_cpu():
    from hartsyinference_b200.models.diffusion.schedulers import FlowUniPCScheduler
    torch.manual_seed(3)
    vs = [torch.randn(2, 16, 8, 8) for _ in range(6)]
    outs = []
    for dev in ("cpu", "cuda"):
        s = FlowUniPCScheduler(6, shift=3.0)
        x = torch.randn(2, 16, 8, 8, generator=torch.Generator().manual_seed(4)).to(dev)
        for v in vs:
            x = s.step(v.to(dev), x)
        outs.append(x.cpu())
    assert (outs[0] - outs[1]).abs().max() < 1e-4
