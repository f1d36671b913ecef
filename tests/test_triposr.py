"""TripoSR: plane lookup + field MLP against torch (CPU), the fused device kernel against the CPU
statement, and the image -> mesh path of the service on a tiny random-init model."""
import pytest
import torch

from hartsyinference_b200.engine.mesh_service import MeshService, prepare_image
from hartsyinference_b200.engine.requests import MeshRequest, Modality, ModelSpec
from hartsyinference_b200.models.threed.triposr import TripoSr, sample_triplane, tiny_triposr


def test_plane_lookup_follows_grid_sample_and_the_axis_pairs():
    torch.manual_seed(0)
    planes = torch.randn(3, 2, 5, 7)
    pts = (torch.rand(50, 3) * 2 - 1) * 0.87
    f = sample_triplane(planes, pts, 0.87)
    assert f.shape == (50, 6)
    # plane 1 reads (x, z): moving y must not change its features
    pts2 = pts.clone()
    pts2[:, 1] = -pts2[:, 1]
    f2 = sample_triplane(planes, pts2, 0.87)
    assert torch.allclose(f[:, 2:4], f2[:, 2:4])
    assert not torch.allclose(f[:, 0:2], f2[:, 0:2])
    # a point in a texel centre returns that texel: x -> width index, y -> height index
    w, h = 7, 5
    cx, cy = 3, 1
    p = torch.tensor([[((2 * cx + 1) / w - 1) * 0.87, ((2 * cy + 1) / h - 1) * 0.87, 0.0]])
    assert torch.allclose(sample_triplane(planes, p, 0.87)[0, :2], planes[0, :, cy, cx], atol=1e-5)


def test_lattice_and_explicit_points_agree_on_cpu():
    m = TripoSr(tiny_triposr())
    planes = torch.randn(3, 8, 8, 8)
    res = 6
    a = m.field(planes, resolution=res)
    ax = torch.linspace(-m.cfg.radius, m.cfg.radius, res)
    pts = torch.stack(torch.meshgrid(ax, ax, ax, indexing="ij"), -1).reshape(-1, 3)
    assert torch.allclose(a, m.field(planes, points=pts), atol=1e-5)


def test_service_builds_a_mesh_file(tmp_path):
    svc = MeshService("cpu")
    img = torch.rand(4, 40, 48)
    img[3] = (torch.arange(40)[:, None] + torch.arange(48)[None] > 30).float()
    out = tmp_path / "m.ply"
    model = svc._model(ModelSpec("synthetic:triposr-tiny", Modality.MESH))
    planes = model.triplane(prepare_image(img, model.cfg.image_size))
    thr = float(model.density(model.field(planes, resolution=12)).median())
    res = svc.run(ModelSpec("synthetic:triposr-tiny", Modality.MESH), MeshRequest(image=img, resolution=12, threshold=thr, output_path=str(out)))
    assert res.vertices.shape[0] > 0 and res.faces.shape[0] > 0 and res.colors.shape == res.vertices.shape
    assert float(res.colors.min()) >= 0 and float(res.colors.max()) <= 1
    assert out.stat().st_size > 100
    assert float(res.vertices.abs().max()) <= model.cfg.radius + 1e-4


@pytest.mark.gpu
@pytest.mark.parametrize("mid", [8, 3, 0])
def test_device_field_kernel_matches_cpu(mid):
    from dataclasses import replace
    torch.manual_seed(1)
    cfg = replace(tiny_triposr(), nerf_mid_layers=mid, triplane_channels=40)
    cpu = TripoSr(cfg, "cpu", seed=3)
    dev = TripoSr(cfg, "cuda", seed=3)
    planes = torch.randn(3, 40, 16, 16)
    want = cpu.field(planes, resolution=20)
    got = dev.field(planes.cuda(), resolution=20)
    assert float((got.cpu() - want).abs().max()) < 2e-3 * float(want.abs().max() + 1)
    pts = (torch.rand(1000, 3) * 2.2 - 1.1) * cfg.radius           # some outside the cube: zero padding
    want = cpu.field(planes, points=pts)
    got = dev.field(planes.cuda(), points=pts.cuda())
    assert float((got.cpu() - want).abs().max()) < 2e-3 * float(want.abs().max() + 1)
