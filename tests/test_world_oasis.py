"""Oasis world model (models/world/oasis.py) and the world service: no released-checkpoint oracle is
available offline, so the tests pin the structure the sampler relies on (causality in time, rotary
tables, the DDIM algebra, patch layouts) and the service / HTTP / CLI plumbing on a tiny random model."""
import base64
import io
import math

import pytest
import torch

from hartsyinference_b200.models.world import oasis as O


def test_rotary_tables():
    a = O.axial_freqs_2d(3, 5, 8, 256.0)
    assert a.shape == (15, 16)
    assert torch.equal(a[:, 0], a[:, 1])                                   # every angle serves a pair of dims
    f = torch.linspace(1.0, 128.0, 4) * math.pi
    assert torch.allclose(a[0 * 5 + 2, :8:2], -1.0 * f) and torch.allclose(a[2 * 5 + 2, :8:2], f)      # rows: -1 .. 1
    assert torch.allclose(a[7, 8::2], torch.linspace(-1, 1, 5)[2] * f)      # columns in the second half
    t = O.temporal_freqs(4, 8)
    assert torch.allclose(t[3, 0::2], 3.0 / (10000.0 ** (torch.arange(0, 8, 2).float() / 8)))
    x = torch.randn(2, 3, 15, 24)
    y = O.apply_rotary(x, a)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5) and torch.equal(y[..., 16:], x[..., 16:])
    # relative property along time: <R(p) q, R(p') k> depends on p - p' only
    q, k = torch.randn(8), torch.randn(8)
    rq = O.apply_rotary(q.expand(4, 8)[None], t)[0]
    rk = O.apply_rotary(k.expand(4, 8)[None], t)[0]
    assert abs(float(rq[3] @ rk[1]) - float(rq[2] @ rk[0])) < 1e-4


def test_denoiser_is_causal_in_time_and_mixes_within_a_frame():
    cfg = O.tiny_oasis()
    dit = O.OasisDit(cfg, "cpu", seed=1)
    torch.manual_seed(0)
    lat = torch.randn(4, 16, 4, 6)
    lv = torch.tensor([14, 14, 14, 500])
    act = torch.randn(4, 25)
    base = dit.forward(lat, lv, act)
    assert base.shape == lat.shape and torch.isfinite(base).all()
    lat2 = lat.clone(); lat2[3] += 1.0
    lv2 = lv.clone(); lv2[3] = 900
    act2 = act.clone(); act2[3] += 1.0
    for changed in (dit.forward(lat2, lv, act), dit.forward(lat, lv2, act), dit.forward(lat, lv, act2)):
        assert torch.allclose(changed[:3], base[:3], atol=1e-5)            # the past does not see the future
        assert not torch.allclose(changed[3], base[3], atol=1e-4)
    lat3 = lat.clone(); lat3[0, :, 0, 0] += 1.0                            # one corner of the first frame ...
    moved = dit.forward(lat3, lv, act)
    assert (moved[0, :, -1, -1] - base[0, :, -1, -1]).abs().max() > 1e-6   # ... reaches the far corner (spatial attention)
    assert (moved[3] - base[3]).abs().max() > 1e-6                         # ... and later frames (temporal attention)
    # a shorter window gives the same prefix
    assert torch.allclose(dit.forward(lat[:2], lv[:2], act[:2]), base[:2], atol=1e-5)


def test_autoencoder_patch_layouts_and_shapes():
    cfg = O.tiny_oasis()
    vae = O.OasisVae(cfg, "cpu", seed=2)
    rgb = torch.rand(1, 3, 8, 12) * 2 - 1
    z = vae.encode(rgb)
    assert z.shape == (1, 16, 2, 3)
    out = vae.decode(z)
    assert out.shape == rgb.shape and torch.isfinite(out).all()
    # the patch embedding is a stride-p convolution with the checkpoint's [width, 3, p, p] kernel
    w = vae.w.linear("patch_embed.proj", cfg.vae_width, 3 * 16)
    conv = torch.nn.functional.conv2d(rgb, w.weight.reshape(cfg.vae_width, 3, 4, 4), w.bias, stride=4)
    p = 4
    x = rgb.reshape(1, 3, 2, p, 3, p).permute(0, 2, 4, 1, 3, 5).reshape(1, 6, 48)
    assert torch.allclose(torch.nn.functional.linear(x, w.weight, w.bias), conv.flatten(2).transpose(1, 2), atol=1e-5)


def test_sampler_schedule_and_ddim_algebra():
    ac = O.sigmoid_alphas_cumprod(1000)
    assert ac.shape == (1000,) and 0.99 < float(ac[0]) <= 1.0 and float(ac[-1]) < 1e-3 and bool((ac[1:] <= ac[:-1]).all())
    cfg = O.tiny_oasis(ddim_steps=4)
    world = O.OasisWorld(cfg, O.OasisDit(cfg, "cpu", seed=1), O.OasisVae(cfg, "cpu", seed=2), seed=5)
    first = world.reset(torch.rand(3, 8, 8))
    assert first.shape == (3, 8, 8) and 0 <= float(first.min()) and float(first.max()) <= 1
    f1 = world.step(torch.zeros(25))
    # context frames sit at the stabilisation level, the new frame walks the schedule downwards
    assert [lv[-1] for lv in world.last_step_levels] == [999, 749, 499, 249] and all(lv[:-1] == [14] for lv in world.last_step_levels)
    f2 = world.step(torch.ones(25))
    assert len(world.frames) == 3 and f2.shape == f1.shape
    # same seed and actions: same world; another action: another frame
    again = O.OasisWorld(cfg, world.dit, world.vae, seed=5)
    again.reset(torch.rand(3, 8, 8, generator=torch.Generator().manual_seed(0)))
    world2 = O.OasisWorld(cfg, world.dit, world.vae, seed=5)
    world2.reset(torch.rand(3, 8, 8, generator=torch.Generator().manual_seed(0)))
    a, b = again.step(torch.zeros(25)), world2.step(torch.zeros(25))
    assert torch.equal(a, b)
    assert not torch.allclose(again.step(torch.ones(25)), world2.step(-torch.ones(25)))
    # the window slides: never more than max_frames frames go through the denoiser
    for _ in range(4):
        world.step(torch.zeros(25))
    assert len(world.last_step_levels[0]) == cfg.max_frames


def test_world_service_sessions_and_http(tmp_path):
    from hartsyinference_b200.engine import InferenceEngine
    from hartsyinference_b200.engine.requests import Modality, ModelSpec, WorldRequest
    eng = InferenceEngine("cpu")
    assert eng.is_supported(Modality.WORLD)
    spec = ModelSpec("synthetic:oasis:tiny", Modality.WORLD)
    pic = (torch.rand(21, 30, 3) * 255).to(torch.uint8)                    # cut to 16 x 24
    sid, first = eng.world.open(spec, pic, seed=1)
    assert first.shape == (3, 16, 24)
    f = eng.world.step(sid, [0.0] * 25)
    assert f.shape == (3, 16, 24) and eng.world.stats(sid)["frames"] == 2
    assert eng.world.close(sid) and not eng.world.close(sid)
    with pytest.raises(KeyError):
        eng.world.step(sid, [0.0] * 25)
    res = eng.world.run(spec, WorldRequest(image=pic, actions=[[0.0] * 25, [1.0] * 25], seed=1))
    assert res.frames.shape == (3, 3, 16, 24) and torch.allclose(res.frames[1], f)
    assert "world:synthetic:oasis:tiny" in eng.loaded_pipeline_keys

    from fastapi.testclient import TestClient
    from PIL import Image
    from hartsyinference_b200.server.app import ServerOptions, create_app
    buf = io.BytesIO()
    Image.fromarray(pic.numpy()).save(buf, format="PNG")
    img = base64.b64encode(buf.getvalue()).decode()
    client = TestClient(create_app(ServerOptions(backend="cpu"), engine=eng))
    r = client.post("/v1/native/world", json={"model": "synthetic:oasis:tiny", "image": img, "seed": 1})
    assert r.status_code == 200, r.text
    sid = r.json()["session"]
    r2 = client.post("/v1/native/world", json={"session": sid, "action": [0.0] * 25})
    assert r2.status_code == 200 and r2.json()["stats"]["frames"] == 2
    png = Image.open(io.BytesIO(base64.b64decode(r2.json()["frame_png_base64"])))
    assert png.size == (24, 16)
    assert client.post("/v1/native/world", json={"session": sid, "close": True}).json() == {"closed": True}
    assert client.post("/v1/native/world", json={"session": sid, "action": [0.0] * 25}).status_code == 404
    r3 = client.post("/v1/native/world", json={"model": "synthetic:oasis:tiny", "image": img, "actions": [[0.0] * 25]})
    assert r3.status_code == 200 and r3.json()["frames"] == 2


@pytest.mark.gpu
def test_gpu_world_steps_and_agrees_with_cpu_on_the_first_frame():
    cfg = O.tiny_oasis(hidden=128, heads=2, vae_width=128)
    pic = torch.rand(3, 16, 24, generator=torch.Generator().manual_seed(0))
    frames = {}
    for dev in ("cpu", "cuda"):
        w = O.OasisWorld(cfg, O.OasisDit(cfg, dev, seed=1), O.OasisVae(cfg, dev, seed=2), seed=3)
        w.reset(pic)
        frames[dev] = torch.stack([w.step(torch.zeros(25)).float().cpu() for _ in range(2)])
    assert torch.isfinite(frames["cuda"]).all()
    # same random weights and noise; the device runs bf16 GEMMs
    assert (frames["cuda"][0] - frames["cpu"][0]).abs().mean() < 0.05
