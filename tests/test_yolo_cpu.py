"""YOLOv8: structure pinned by the published parameter counts of the five sizes, BatchNorm folding, box decoding
against a plain restatement, letterbox geometry and the vision service's detect route."""
import json

import pytest
import torch
import torch.nn.functional as F

from hartsyinference_b200.models.vision.yolo import REG_MAX, YoloV8, detect_size, yolo_config

PUBLISHED = {"n": 3157200, "s": 11166560, "m": 25902640, "l": 43691520, "x": 68229648}


@pytest.mark.parametrize("size", ["n", "s", "m", "l", "x"])
def test_parameter_count_matches_the_published_model(size):
    m = YoloV8(yolo_config(size), "cpu")
    boxes, scores = m.forward(torch.rand(1, 3, 64, 96))
    assert m.param_count_total == PUBLISHED[size]
    cells = (64 // 8) * (96 // 8) + (64 // 16) * (96 // 16) + (64 // 32) * (96 // 32)
    assert boxes.shape == (1, cells, 4) and scores.shape == (1, cells, 80)
    assert float(scores.min()) >= 0 and float(scores.max()) <= 1


PUBLISHED_11 = {"n": 2624080, "s": 9458752, "m": 20114688, "l": 25372160, "x": 56966176}


def _count(**kw):
    m = YoloV8(yolo_config(**kw), "meta")
    out = m.forward_all(torch.empty(1, 3, 64, 64, device="meta"))
    return m.param_count_total, {k: tuple(v.shape) for k, v in out.items()}


@pytest.mark.parametrize("size", ["n", "s", "m", "l", "x"])
def test_yolo11_parameter_count_matches_the_published_model(size):
    assert _count(size=size, arch="11")[0] == PUBLISHED_11[size]


def test_segment_and_pose_heads_match_the_published_models():
    n, shapes = _count(size="n", task="segment")
    assert n == 3409968 and shapes["coefficients"] == (1, 84, 32) and shapes["prototypes"] == (1, 32, 16, 16)
    n, shapes = _count(size="n", task="pose", num_classes=1)
    assert n == 3295470 and shapes["keypoints"] == (1, 84, 17, 3)
    assert _count(size="n", arch="11", task="segment")[0] == 2876848
    assert _count(size="n", arch="11", task="pose", num_classes=1)[0] == 2874462
    assert _count(size="n", task="pose", num_classes=1, keypoints=5, kpt_dims=2)[1]["keypoints"] == (1, 84, 5, 2)


def _unfolded_state(cfg, seed=1):
    """A random checkpoint with separate BatchNorm statistics, by the trainer's tensor names."""
    probe = YoloV8(cfg, "cpu")
    probe.forward(torch.rand(1, 3, 32, 32))
    g = torch.Generator().manual_seed(seed)
    sd = {}
    for name, (w, b) in probe._w.items():
        if name.endswith(".proto.upsample"):
            sd[name + ".weight"], sd[name + ".bias"] = torch.randn(w.shape, generator=g) * 0.1, torch.randn(b.shape, generator=g) * 0.1
            continue
        if name.endswith(".2") and (".cv2." in name or ".cv3." in name or ".cv4." in name):
            sd[name + ".weight"], sd[name + ".bias"] = torch.randn(w.shape, generator=g) * 0.1, torch.randn(b.shape, generator=g) * 0.1
            continue
        co = w.shape[0]
        sd[name + ".conv.weight"] = torch.randn(w.shape, generator=g) * (1.0 / w[0].numel()) ** 0.5
        sd[name + ".bn.weight"] = torch.rand(co, generator=g) + 0.5
        sd[name + ".bn.bias"] = torch.randn(co, generator=g) * 0.1
        sd[name + ".bn.running_mean"] = torch.randn(co, generator=g) * 0.1
        sd[name + ".bn.running_var"] = torch.rand(co, generator=g) + 0.5
    return sd


def _plain_forward(sd, cfg, x):
    """The network written out with separate BatchNorm layers (eval mode), in the layer order of the definition file."""
    def conv(t, p, k=1, s=1):
        t = F.conv2d(t, sd[p + ".conv.weight"], None, s, k // 2)
        t = F.batch_norm(t, sd[p + ".bn.running_mean"], sd[p + ".bn.running_var"], sd[p + ".bn.weight"], sd[p + ".bn.bias"], False, 0.0, 1e-3)
        return t * torch.sigmoid(t)

    def c2f(t, p, n, shortcut):
        y = list(conv(t, p + ".cv1").chunk(2, 1))
        for i in range(n):
            h = conv(conv(y[-1], f"{p}.m.{i}.cv1", 3), f"{p}.m.{i}.cv2", 3)
            y.append(y[-1] + h if shortcut else h)
        return conv(torch.cat(y, 1), p + ".cv2")

    r = cfg.reps
    t = conv(x, "model.0", 3, 2); t = conv(t, "model.1", 3, 2); t = c2f(t, "model.2", r(3), True)
    t = conv(t, "model.3", 3, 2); p3 = c2f(t, "model.4", r(6), True)
    t = conv(p3, "model.5", 3, 2); p4 = c2f(t, "model.6", r(6), True)
    t = conv(p4, "model.7", 3, 2); t = c2f(t, "model.8", r(3), True)
    a = conv(t, "model.9.cv1"); b = F.max_pool2d(a, 5, 1, 2); c = F.max_pool2d(b, 5, 1, 2); d = F.max_pool2d(c, 5, 1, 2)
    p5 = conv(torch.cat([a, b, c, d], 1), "model.9.cv2")
    up = torch.nn.Upsample(scale_factor=2, mode="nearest")
    n4 = c2f(torch.cat([up(p5), p4], 1), "model.12", r(3), False)
    n3 = c2f(torch.cat([up(n4), p3], 1), "model.15", r(3), False)
    d4 = c2f(torch.cat([conv(n3, "model.16", 3, 2), n4], 1), "model.18", r(3), False)
    d5 = c2f(torch.cat([conv(d4, "model.19", 3, 2), p5], 1), "model.21", r(3), False)
    boxes, scores = [], []
    for i, f in enumerate([n3, d4, d5]):
        stride = x.shape[-1] // f.shape[-1]
        reg = F.conv2d(conv(conv(f, f"model.22.cv2.{i}.0", 3), f"model.22.cv2.{i}.1", 3), sd[f"model.22.cv2.{i}.2.weight"], sd[f"model.22.cv2.{i}.2.bias"])
        cls = F.conv2d(conv(conv(f, f"model.22.cv3.{i}.0", 3), f"model.22.cv3.{i}.1", 3), sd[f"model.22.cv3.{i}.2.weight"], sd[f"model.22.cv3.{i}.2.bias"])
        _, _, h, w = f.shape
        for yy in range(h):
            for xx in range(w):
                dist = [float((reg[0, s * REG_MAX:(s + 1) * REG_MAX, yy, xx].softmax(0) * torch.arange(REG_MAX)).sum()) for s in range(4)]
                boxes.append([(xx + 0.5 - dist[0]) * stride, (yy + 0.5 - dist[1]) * stride, (xx + 0.5 + dist[2]) * stride, (yy + 0.5 + dist[3]) * stride])
                scores.append(cls[0, :, yy, xx].sigmoid())
    return torch.tensor(boxes), torch.stack(scores)


def test_batchnorm_folding_and_decoding_match_the_layerwise_network():
    cfg = yolo_config("n", num_classes=5)
    sd = _unfolded_state(cfg)
    assert detect_size(sd.get) == cfg
    m = YoloV8(cfg, "cpu", get=sd.get)
    x = torch.rand(1, 3, 64, 64)
    boxes, scores = m.forward(x)
    want_b, want_s = _plain_forward(sd, cfg, x)
    assert torch.allclose(boxes[0], want_b, atol=2e-3), float((boxes[0] - want_b).abs().max())
    assert torch.allclose(scores[0], want_s, atol=1e-4)


def test_detect_size_tells_architectures_sizes_and_tasks_apart():
    cases = [dict(size=s, arch=a) for s in "nsmlx" for a in ("v8", "11")]
    cases += [dict(size="s", task="segment"), dict(size="n", arch="11", task="pose", num_classes=1),
              dict(size="m", task="pose", num_classes=1, keypoints=5, kpt_dims=2)]
    for kw in cases:
        cfg = yolo_config(**{"num_classes": 3, **kw})
        probe = YoloV8(cfg, "meta")
        probe.forward_all(torch.empty(1, 3, 32, 32, device="meta"))
        shapes = {}
        for k, (w, b) in probe._w.items():
            plain = k.endswith(".proto.upsample") or (k.endswith(".2") and any(t in k for t in (".cv2.", ".cv3.", ".cv4.")))
            shapes[(k + ".weight") if plain else (k + ".conv.weight")] = w
        assert detect_size(shapes.get) == cfg, kw


def test_pose_and_mask_decoding():
    cfg = yolo_config("n", num_classes=1, task="pose", keypoints=5)
    sd = _unfolded_state(cfg, seed=2)
    m = YoloV8(cfg, "cpu", get=sd.get)
    x = torch.rand(1, 3, 64, 64)
    out = m.forward_all(x)
    # first stride-8 cell (0, 0): keypoint = (2 v + cell index) x 8
    feats = m.features(x)
    raw = m._branch(feats[0], "model.22.cv4.0", max(feats[0].shape[1] // 4, 15), 15)[0, :, 0, 1].view(5, 3)
    want = torch.stack([(raw[:, 0] * 2 + 1) * 8, (raw[:, 1] * 2 + 0) * 8, raw[:, 2].sigmoid()], 1)
    assert torch.allclose(out["keypoints"][0, 1], want, atol=1e-5)

    cfg = yolo_config("n", num_classes=2, task="segment")
    sd = _unfolded_state(cfg, seed=3)
    for i in range(3):
        sd[f"model.22.cv3.{i}.2.bias"] = torch.tensor([1.5, -4.0])
    m = YoloV8(cfg, "cpu", get=sd.get)
    found = m.detect(x, 0.3, 0.5, full=True)[0]
    assert found and found[0]["mask"].shape == (64, 64) and found[0]["mask"].dtype == torch.bool
    x0, y0, x1, y1 = found[0]["box"]
    ys, xs = found[0]["mask"].nonzero(as_tuple=True)
    if len(xs):                                                # nothing of the mask lies outside its box
        assert xs.min() >= int(max(x0, 0)) and xs.max() <= int(x1) + 1 and ys.min() >= int(max(y0, 0)) and ys.max() <= int(y1) + 1


def test_yolo11_attention_block_is_a_softmax_over_positions():
    """C2PSA on a constant map: every position attends uniformly, so the block's output is constant too."""
    m = YoloV8(yolo_config("n", arch="11"), "cpu")
    x = torch.ones(1, 256, 4, 4) * 0.3
    y = m._c2psa(x, "model.10", 1)
    inner = y[:, :, 1:3, 1:3]
    assert torch.allclose(inner, inner[:, :, :1, :1].expand_as(inner), atol=1e-5)


def test_letterbox_round_trip():
    from hartsyinference_b200.engine.vision_service import letterbox
    img = torch.rand(3, 100, 200)
    sq, scale, (px, py) = letterbox(img, 64)
    assert sq.shape == (3, 64, 64) and abs(scale - 0.32) < 1e-9 and px == 0 and py == 16
    assert torch.allclose(sq[:, :py], torch.full((3, py, 64), 114 / 255))
    x, y = 150.0, 40.0
    assert abs((x * scale + px - px) / scale - x) < 1e-6 and abs((y * scale + py - py) / scale - y) < 1e-6


def test_vision_service_detects_with_a_yolo_checkpoint(tmp_path):
    from hartsyinference_b200.assets.safetensors import save_file
    from hartsyinference_b200.engine.requests import ModelSpec, VisionRequest
    from hartsyinference_b200.engine.vision_service import VisionService, letterbox
    cfg = yolo_config("n", num_classes=3)
    sd = _unfolded_state(cfg, seed=4)
    for i in range(3):                                       # confident head so that something is found
        sd[f"model.22.cv3.{i}.2.bias"] = torch.tensor([2.0, -4.0, -4.0])
    save_file({k: v.contiguous() for k, v in sd.items()}, tmp_path / "yolo.safetensors")
    (tmp_path / "config.json").write_text(json.dumps({"model_type": "yolov8", "names": ["cat", "dog", "bird"], "image_size": 64}))
    svc = VisionService("cpu")
    img = (torch.rand(48, 96, 3) * 255).to(torch.uint8)
    spec = ModelSpec(str(tmp_path))
    res = svc.run(spec, VisionRequest(operation="detect", images=[img], score_threshold=0.3, nms_iou=0.5))
    found = res.detections[0]
    assert found and all(d["label"] in ("cat", "dog", "bird") for d in found)
    assert all(0 <= d["box"][0] <= d["box"][2] <= 96 and 0 <= d["box"][1] <= d["box"][3] <= 48 for d in found)
    # the same boxes straight from the model, mapped back through the letterbox
    sq, scale, (px, py) = letterbox(img.permute(2, 0, 1).float() / 255, 64)
    direct = YoloV8(cfg, "cpu", get=sd.get).detect(sq[None], 0.3, 0.5)[0]
    assert len(direct) == len(found) and abs(direct[0][1] - found[0]["score"]) < 1e-5
    only = svc.run(spec, VisionRequest(operation="detect", images=[img], texts=["dog"], score_threshold=0.3)).detections[0]
    assert all(d["label"] == "dog" for d in only)
    with pytest.raises(ValueError):
        svc.run(spec, VisionRequest(operation="embed", images=[img]))
