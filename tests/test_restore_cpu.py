"""Real-ESRGAN: the network against the canonical module layout, tiling, service, endpoint, CLI."""
import base64
import io

import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

from hartsyinference_b200.models.vision.rrdbnet import RrdbConfig, RrdbNet, UpscalePipeline, detect_rrdb_config


class _Rdb(nn.Module):
    def __init__(self, nf, gc):
        super().__init__()
        for i in range(1, 6):
            setattr(self, f"conv{i}", nn.Conv2d(nf + (i - 1) * gc, gc if i < 5 else nf, 3, 1, 1))

    def forward(self, x):
        x1 = F.leaky_relu(self.conv1(x), 0.2)
        x2 = F.leaky_relu(self.conv2(torch.cat((x, x1), 1)), 0.2)
        x3 = F.leaky_relu(self.conv3(torch.cat((x, x1, x2), 1)), 0.2)
        x4 = F.leaky_relu(self.conv4(torch.cat((x, x1, x2, x3), 1)), 0.2)
        return self.conv5(torch.cat((x, x1, x2, x3, x4), 1)) * 0.2 + x


class _Rrdb(nn.Module):
    def __init__(self, nf, gc):
        super().__init__()
        self.rdb1, self.rdb2, self.rdb3 = _Rdb(nf, gc), _Rdb(nf, gc), _Rdb(nf, gc)

    def forward(self, x):
        return self.rdb3(self.rdb2(self.rdb1(x))) * 0.2 + x


class _Net(nn.Module):
    """The published module layout, restated: its state dict is what a release file holds."""

    def __init__(self, nf, nb, gc, scale):
        super().__init__()
        self.scale = scale
        self.conv_first = nn.Conv2d(3 * (4 if scale == 2 else 1), nf, 3, 1, 1)
        self.body = nn.Sequential(*[_Rrdb(nf, gc) for _ in range(nb)])
        self.conv_body, self.conv_up1, self.conv_up2 = (nn.Conv2d(nf, nf, 3, 1, 1) for _ in range(3))
        self.conv_hr, self.conv_last = nn.Conv2d(nf, nf, 3, 1, 1), nn.Conv2d(nf, 3, 3, 1, 1)

    def forward(self, x):
        feat = self.conv_first(F.pixel_unshuffle(x, 2) if self.scale == 2 else x)
        feat = feat + self.conv_body(self.body(feat))
        feat = F.leaky_relu(self.conv_up1(F.interpolate(feat, scale_factor=2, mode="nearest")), 0.2)
        feat = F.leaky_relu(self.conv_up2(F.interpolate(feat, scale_factor=2, mode="nearest")), 0.2)
        return self.conv_last(F.leaky_relu(self.conv_hr(feat), 0.2))


@pytest.mark.parametrize("scale", [4, 2])
def test_rrdbnet_matches_the_module_layout(scale):
    torch.manual_seed(0)
    ref = _Net(16, 3, 8, scale).eval()
    sd = {"params_ema." + k: v.detach() for k, v in ref.state_dict().items()}
    assert detect_rrdb_config(sd.keys()).num_block == 3
    net = RrdbNet(RrdbConfig(16, 3, 8, scale), "cpu", get=sd.get)
    assert net.scale == scale
    x = torch.rand(1, 3, 24, 32)
    with torch.no_grad():
        want = ref(x)
    got = net.forward(x)
    assert got.shape == (1, 3, 24 * scale, 32 * scale) and torch.allclose(got, want, atol=1e-5)


def test_tiled_upscale_blends_to_the_whole_image_result():
    torch.manual_seed(1)
    ref = _Net(16, 1, 8, 4).eval()
    net = RrdbNet(RrdbConfig(16, 1, 8, 4), "cpu", get={k: v.detach() for k, v in ref.state_dict().items()}.get)
    img = torch.rand(3, 50, 70)
    whole = UpscalePipeline(net, tile=0).upscale_tensor(img)
    tiled = UpscalePipeline(net, tile=32, overlap=0.5).upscale_tensor(img)
    assert whole.shape == tiled.shape == (3, 200, 280)
    # tiles see a truncated neighbourhood near their borders; the ramps keep the seams small
    assert (whole - tiled).abs().mean() < 5e-3 and (whole - tiled).abs().max() < 0.2
    rgb, w, h = UpscalePipeline(net, tile=0).upscale_rgb(bytes(range(48)) * 4, 8, 8)
    assert (w, h) == (32, 32) and len(rgb) == 32 * 32 * 3
    odd = UpscalePipeline(RrdbNet(RrdbConfig(8, 1, 4, 2), "cpu"), tile=0).upscale_tensor(torch.rand(3, 9, 11))
    assert odd.shape == (3, 18, 22)


def test_restore_service_endpoint_and_cli(tmp_path):
    from click.testing import CliRunner
    from fastapi.testclient import TestClient
    from PIL import Image
    from hartsyinference_b200.assets.safetensors import save_file
    from hartsyinference_b200.cli.main import cli
    from hartsyinference_b200.engine import InferenceEngine, ModelSpec, RestoreRequest
    from hartsyinference_b200.engine.requests import Modality
    from hartsyinference_b200.server.app import ServerOptions, create_app
    torch.manual_seed(2)
    ref = _Net(8, 2, 4, 4)
    save_file({k: v.detach().contiguous() for k, v in ref.state_dict().items()}, tmp_path / "esrgan.safetensors")
    torch.save({"params_ema": ref.state_dict()}, tmp_path / "esrgan.pth")
    eng = InferenceEngine("cpu")
    assert eng.is_supported(Modality.RESTORE)
    img = torch.rand(3, 20, 28)
    a = eng.restore.run(ModelSpec(str(tmp_path / "esrgan.safetensors")), RestoreRequest(image=img, tile=0))
    b = eng.restore.run(ModelSpec(str(tmp_path / "esrgan.pth")), RestoreRequest(image=img, tile=0))
    assert (a.width, a.height) == (112, 80) and a.rgb == b.rgb and a.meta["scale"] == 4
    with pytest.raises(ValueError):
        eng.restore.run(ModelSpec(str(tmp_path / "esrgan.pth")), RestoreRequest(operation="deblur", image=img))
    pil = Image.fromarray((img.permute(1, 2, 0) * 255).byte().numpy())
    buf = io.BytesIO()
    pil.save(buf, format="PNG")
    pil.save(tmp_path / "in.png")
    app = create_app(ServerOptions(models={"up": str(tmp_path / "esrgan.safetensors")}), engine=eng)
    with TestClient(app) as c:
        r = c.post("/v1/native/restore", json={"model": "up", "image": base64.b64encode(buf.getvalue()).decode(), "tile": 16})
        assert r.status_code == 200, r.text
        j = r.json()
        assert (j["width"], j["height"]) == (112, 80)
        assert Image.open(io.BytesIO(base64.b64decode(j["png_base64"]))).size == (112, 80)
        assert c.post("/v1/native/restore", json={"model": "up"}).status_code == 400
    eng.close()
    r = CliRunner().invoke(cli, ["restore", str(tmp_path / "esrgan.safetensors"), str(tmp_path / "in.png"),
                                 "--out", str(tmp_path / "o.png"), "--device", "cpu"])
    assert r.exit_code == 0, r.output
    assert Image.open(tmp_path / "o.png").size == (112, 80)
