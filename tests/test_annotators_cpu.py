"""Control-image annotators: edge detection on synthetic shapes, skeleton drawing, depth / label pictures."""
import torch

from hartsyinference_b200.models.vision import annotators as A


def test_canny_finds_the_outline_of_a_square_and_nothing_else():
    img = torch.zeros(3, 64, 64)
    img[:, 16:48, 20:44] = 1.0
    e = A.canny(img)
    assert e.dtype == torch.bool and e.shape == (64, 64)
    ys, xs = e.nonzero(as_tuple=True)
    assert 80 < len(ys) < 260                                   # a thin outline: perimeter 112, at most two pixels wide
    on_border = ((ys - 16).abs() <= 2) | ((ys - 47).abs() <= 2) | ((xs - 20).abs() <= 2) | ((xs - 43).abs() <= 2)
    assert bool(on_border.all())
    assert not bool(e[28:36, 28:36].any()) and not bool(e[:8].any())
    assert not bool(A.canny(torch.full((3, 32, 32), 0.5)).any())     # flat picture: no edges
    # a faint step is dropped by the thresholds, and kept when they are lowered
    faint = torch.zeros(3, 32, 32)
    faint[:, :, 16:] = 0.05
    assert not bool(A.canny(faint).any()) and bool(A.canny(faint, 5, 10).any())
    # hysteresis: along one edge whose contrast fades from 1.0 to 0.1 the weak end survives because it is chained to
    # the strong end; the same weak end on its own (the picture cropped to it) has nothing to hold on to
    fade = torch.ones(3, 40, 80)
    fade[:, :20] = (torch.arange(80) * 0.9 / 79)[None, None, :]
    e = A.canny(fade, 30, 200)
    assert bool(e[18:22, 5:15].any()) and bool(e[18:22, 70:78].any())
    assert not bool(A.canny(fade[:, :, 64:], 30, 200).any())


def test_pose_rendering():
    kp = torch.zeros(17, 3)
    pts = {0: (50, 20), 5: (60, 40), 6: (40, 40), 7: (70, 60), 8: (30, 60), 9: (75, 80), 10: (25, 80), 11: (58, 90), 12: (42, 90),
           13: (60, 120), 14: (40, 120), 15: (60, 150), 16: (40, 150)}
    for i, (x, y) in pts.items():
        kp[i] = torch.tensor([x, y, 0.9])
    b = A.body18(kp)
    assert b[1, :2].tolist() == [50.0, 40.0] and b[1, 2] == 1 and b[14, 2] == 0            # neck between the shoulders; no eyes given
    pic = A.render_pose([kp], 160, 100)
    assert pic.shape == (160, 100, 3) and pic.dtype == torch.uint8
    assert pic[40, 50].sum() > 0 and pic[105, 59].sum() > 0 and pic[5, 5].sum() == 0         # shoulder line, a thigh, empty corner
    assert tuple(pic[20, 50].tolist()) == A.COLOURS[0]                                        # the nose joint in its colour
    hidden = kp.clone()
    hidden[13:, 2] = 0.1
    assert A.render_pose([hidden], 160, 100)[135, 60].sum() == 0                              # unseen joints draw nothing


def test_depth_label_and_tile_pictures():
    d = torch.linspace(2.0, 10.0, 12).view(3, 4)
    g = A.depth_control(d)
    assert g.shape == (3, 4, 3) and g[0, 0, 0] == 0 and g[2, 3, 0] == 255 and bool((g[..., 0] == g[..., 2]).all())
    pal = A.label_palette(torch.tensor([[0, 1, 2], [3, 8, 15]]))
    assert pal[0, 0].tolist() == [0, 0, 0] and pal[0, 1].tolist() == [128, 0, 0] and pal[0, 2].tolist() == [0, 128, 0]
    assert pal[1, 0].tolist() == [128, 128, 0] and pal[1, 1].tolist() == [64, 0, 0]
    img = torch.rand(3, 32, 48)
    px = A.pixelate(img, 8)
    assert px.shape == img.shape and torch.allclose(px[:, :8, :8], img[:, :8, :8].mean((1, 2))[:, None, None].expand(3, 8, 8), atol=1e-6)
    bl = A.tile_blur(img, 2.0)
    assert bl.shape == img.shape and float(bl.std()) < float(img.std()) and abs(float(bl.mean()) - float(img.mean())) < 0.02


def test_annotate_operation_of_the_vision_service(tmp_path):
    import json
    import pytest
    from hartsyinference_b200.assets.safetensors import save_file
    from hartsyinference_b200.engine.requests import ModelSpec, VisionRequest
    from hartsyinference_b200.engine.vision_service import VisionService
    from hartsyinference_b200.models.vision.yolo import YoloV8, yolo_config
    svc = VisionService("cpu")
    img = torch.zeros(48, 64, 3, dtype=torch.uint8)
    img[12:36, 16:48] = 255
    res = svc.run(ModelSpec("none"), VisionRequest(operation="annotate", annotator="canny", images=[img]))
    edge = res.control_images[0]
    assert edge.shape == (48, 64, 3) and edge.dtype == torch.uint8 and 0 < int((edge[..., 0] > 0).sum()) < 400
    assert svc.run(ModelSpec("none"), VisionRequest(operation="annotate", annotator="tile", images=[img])).control_images[0].shape == (48, 64, 3)
    with pytest.raises(ValueError):
        svc.run(ModelSpec("none"), VisionRequest(operation="annotate", annotator="scribble", images=[img]))
    # pose: a tiny pose checkpoint whose class head is confident everywhere
    cfg = yolo_config("n", num_classes=1, task="pose")
    probe = YoloV8(cfg, "cpu", seed=3)
    probe.forward_all(torch.rand(1, 3, 64, 64))
    sd = {}
    for name, (w, b) in probe._w.items():
        plain = name.endswith(".2") and any(t in name for t in (".cv2.", ".cv3.", ".cv4."))
        sd[name + (".weight" if plain else ".conv.weight")] = w.reshape(w.shape[0], -1, 1, 1).contiguous() if plain else w.contiguous()
        sd[name + (".bias" if plain else ".conv.bias")] = (torch.full_like(b, 3.0) if plain and ".cv3." in name else b).contiguous()
    save_file(sd, tmp_path / "pose.safetensors")
    (tmp_path / "config.json").write_text(json.dumps({"model_type": "yolov8", "image_size": 64}))
    res = svc.run(ModelSpec(str(tmp_path)), VisionRequest(operation="annotate", annotator="pose", images=[img], score_threshold=0.5, nms_iou=0.3))
    assert res.control_images[0].shape == (48, 64, 3) and res.control_images[0].dtype == torch.uint8
    with pytest.raises(ValueError):
        svc.run(ModelSpec(str(tmp_path)), VisionRequest(operation="annotate", annotator="depth", images=[img]))


def test_vision_route_returns_control_images_and_label_maps(tmp_path):
    import base64
    import io
    import json
    import pytest
    pytest.importorskip("fastapi")
    from fastapi.testclient import TestClient
    from PIL import Image
    from hartsyinference_b200.assets.safetensors import save_file
    from hartsyinference_b200.engine import InferenceEngine
    from hartsyinference_b200.server.app import ServerOptions, create_app
    import os
    import sys
    sys.path.insert(0, os.path.dirname(__file__))
    from test_upernet_cpu import _tiny
    cfg, model = _tiny()
    raw = cfg.to_dict()
    raw["model_type"] = "upernet"
    raw["short_side"] = 64
    d = tmp_path / "scene"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(raw, default=str))
    save_file({k: v.contiguous() for k, v in model.state_dict().items() if not k.endswith("num_batches_tracked")}, d / "model.safetensors")
    pic = torch.zeros(40, 56, 3, dtype=torch.uint8)
    pic[10:30, 12:40] = 255
    buf = io.BytesIO()
    Image.fromarray(pic.numpy()).save(buf, format="PNG")
    b64 = base64.b64encode(buf.getvalue()).decode()
    eng = InferenceEngine("cpu")
    with TestClient(create_app(ServerOptions(models={"scene": str(d)}), engine=eng)) as cl:
        r = cl.post("/v1/native/vision", json={"model": "scene", "operation": "annotate", "annotator": "canny", "images": [b64]})
        assert r.status_code == 200, r.text
        c = r.json()["control_images"][0]
        edge = Image.open(io.BytesIO(base64.b64decode(c["png_base64"])))
        assert (c["width"], c["height"]) == (56, 40) and edge.size == (56, 40) and edge.getbbox() is not None
        r = cl.post("/v1/native/vision", json={"model": "scene", "operation": "segment", "images": [b64]})
        assert r.status_code == 200, r.text
        m = r.json()["label_maps"][0]
        assert (m["width"], m["height"]) == (56, 40) and m["labels"] and Image.open(io.BytesIO(base64.b64decode(m["png_base64"]))).size == (56, 40)
        r = cl.post("/v1/native/vision", json={"model": "scene", "operation": "annotate", "annotator": "segmentation", "images": [b64]})
        assert r.status_code == 200 and r.json()["control_images"][0]["width"] == 56
    eng.close()
