"""UperNet (Swin backbone) against `transformers.UperNetForSemanticSegmentation` with tiny random weights."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from hartsyinference_b200.models.vision.upernet import UperNet, UperNetConfig  # noqa: E402


def _tiny():
    torch.manual_seed(0)
    swin = transformers.SwinConfig(embed_dim=16, depths=[2, 2, 2, 2], num_heads=[2, 2, 4, 4], window_size=4,
                                   out_features=["stage1", "stage2", "stage3", "stage4"], drop_path_rate=0.0)
    cfg = transformers.UperNetConfig(backbone_config=swin, hidden_size=32, num_labels=7, use_auxiliary_head=False)
    model = transformers.UperNetForSemanticSegmentation(cfg).eval()
    with torch.no_grad():
        for n, b in model.named_buffers():
            if n.endswith("running_mean"):
                b.normal_(0, 0.2)
            elif n.endswith("running_var"):
                b.uniform_(0.5, 1.5)
    return cfg, model


def test_logits_match_transformers():
    cfg, model = _tiny()
    x = torch.randn(1, 3, 96, 128)
    with torch.no_grad():
        want = model(pixel_values=x).logits
    mine = UperNet(UperNetConfig.from_hf(cfg.to_dict()), model.state_dict().get)
    got = mine.logits(x)
    assert got.shape == want.shape == (1, 7, 96, 128) and torch.allclose(got, want, atol=5e-4), float((got - want).abs().max())
    assert torch.equal(mine.segment(x), want.argmax(1)) or (mine.segment(x) == want.argmax(1)).float().mean() > 0.999


def test_vision_service_segments_scenes(tmp_path):
    import json
    from hartsyinference_b200.assets.safetensors import save_file
    from hartsyinference_b200.engine.requests import ModelSpec, VisionRequest
    from hartsyinference_b200.engine.vision_service import VisionService
    cfg, model = _tiny()
    raw = cfg.to_dict()
    raw["model_type"] = "upernet"
    raw["id2label"] = {str(i): n for i, n in enumerate(["wall", "floor", "tree", "sky", "road", "car", "person"])}
    (tmp_path / "config.json").write_text(json.dumps(raw, default=str))
    save_file({k: v.contiguous() for k, v in model.state_dict().items() if not k.endswith("num_batches_tracked")}, tmp_path / "model.safetensors")
    svc = VisionService("cpu")
    img = (torch.rand(64, 80, 3) * 255).to(torch.uint8)
    res = svc.run(ModelSpec(str(tmp_path)), VisionRequest(operation="segment", images=[img]))
    labels = res.masks[0]
    assert labels.shape == (64, 80) and labels.dtype == torch.int64 and int(labels.max()) < 7
    assert set(res.labels[0]) <= {"wall", "floor", "tree", "sky", "road", "car", "person"}
    with pytest.raises(ValueError):
        svc.run(ModelSpec(str(tmp_path)), VisionRequest(operation="detect", images=[img], texts=["x"]))
