"""SAM 2 image segmentation (models/vision/sam2.py) against ``transformers.Sam2Model`` with random tiny
weights: point, box, point + box and mask prompts, several prompts per image, single-mask selection."""
import pytest
import torch

from hartsyinference_b200.models.vision.sam2 import Sam2, sam2_from_hf


def _hf(seed=0):
    from transformers import Sam2Config, Sam2Model
    from transformers.models.sam2.configuration_sam2 import (Sam2HieraDetConfig, Sam2MaskDecoderConfig, Sam2PromptEncoderConfig,
                                                             Sam2VisionConfig)
    torch.manual_seed(seed)
    bb = Sam2HieraDetConfig(hidden_size=16, num_attention_heads=1, image_size=[64, 64], blocks_per_stage=[1, 2, 3, 2],
                            embed_dim_per_stage=[16, 32, 64, 128], num_attention_heads_per_stage=[1, 2, 4, 8],
                            window_size_per_stage=[8, 4, 6, 4], global_attention_blocks=[4, 5])
    vc = Sam2VisionConfig(backbone_config=bb, backbone_channel_list=[128, 64, 32, 16], backbone_feature_sizes=[[16, 16], [8, 8], [4, 4]],
                          fpn_hidden_size=32)
    c = Sam2Config(vision_config=vc,
                   prompt_encoder_config=Sam2PromptEncoderConfig(hidden_size=32, image_size=64, patch_size=16, mask_input_channels=16),
                   mask_decoder_config=Sam2MaskDecoderConfig(hidden_size=32, mlp_dim=64, num_attention_heads=2, iou_head_hidden_dim=32))
    m = Sam2Model(c).eval()
    with torch.no_grad():                       # zero-initialised tables would hide indexing mistakes
        for n, p in m.named_parameters():
            if "pos_embed" in n or "no_memory" in n or n.endswith("embed.weight") or "token" in n:
                p.normal_(0, 0.5)
    return c, m


def test_matches_transformers():
    c, hf = _hf()
    sd = hf.state_dict()
    mine = Sam2(sam2_from_hf(c.to_dict()), "cpu", get=sd.get)
    x = torch.randn(2, 3, 64, 64)
    maps = mine.image_embeddings(x)
    with torch.no_grad():
        want_maps = hf.get_image_embeddings(x)
    for a, b in zip(maps, want_maps):
        assert a.shape == b.shape and (a - b).abs().max() < 2e-4 * max(1.0, float(b.abs().max()))
    pts = torch.tensor([[[[20.0, 30.0], [40.0, 12.0]], [[5.0, 50.0], [0.0, 0.0]]],
                        [[[33.0, 33.0], [10.0, 10.0]], [[60.0, 2.0], [7.0, 7.0]]]])           # [2 images, 2 prompts, 2 points, 2]
    lab = torch.tensor([[[1, 0], [1, -10]], [[1, 1], [0, 1]]])
    boxes = torch.tensor([[[10.0, 12.0, 40.0, 50.0], [0.0, 0.0, 63.0, 63.0]], [[5.0, 5.0, 20.0, 30.0], [30.0, 10.0, 50.0, 60.0]]])
    mask_in = torch.randn(2, 1, 64, 64)
    cases = [dict(input_points=pts, input_labels=lab), dict(input_boxes=boxes), dict(input_points=pts, input_labels=lab, input_boxes=boxes),
             dict(input_points=pts[:, :1], input_labels=lab[:, :1], input_masks=mask_in), dict()]
    for kw in cases:
        for multi in (True, False):
            with torch.no_grad():
                want = hf(pixel_values=x, multimask_output=multi, **kw)
            got = mine.predict(maps, kw.get("input_points"), kw.get("input_labels"), kw.get("input_boxes"), kw.get("input_masks"), multi)
            assert got[0].shape == want.pred_masks.shape, (kw.keys(), multi)
            scale = max(1.0, float(want.pred_masks.abs().max()))
            assert (got[0] - want.pred_masks).abs().max() < 5e-4 * scale, (list(kw), multi)
            assert (got[1] - want.iou_scores).abs().max() < 1e-4
            assert (got[2] - want.object_score_logits).abs().max() < 1e-3


def test_vision_service_segments_from_points_and_boxes(tmp_path):
    import json
    from hartsyinference_b200.assets.safetensors import save_file
    from hartsyinference_b200.engine import InferenceEngine
    from hartsyinference_b200.engine.requests import ModelSpec, VisionRequest
    c, hf = _hf(1)
    d = tmp_path / "sam2"
    d.mkdir()
    cfg = c.to_dict()
    cfg["model_type"] = "sam2"
    (d / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.contiguous() for k, v in hf.state_dict().items()}, d / "model.safetensors")
    eng = InferenceEngine("cpu")
    pic = torch.rand(3, 48, 80)
    req = VisionRequest(operation="segment", images=[pic], points=[[[10, 12], [60, 40]], [[30, 30]]], point_labels=[[1, 0]])
    res = eng.vision.run(ModelSpec(str(d)), req)
    assert res.masks[0].shape == (2, 48, 80) and 0 <= float(res.masks[0].min()) and float(res.masks[0].max()) <= 1
    assert res.mask_scores[0].shape == (2,)
    # against transformers on the same squeezed, normalised picture: the second prompt (one foreground point)
    x = torch.nn.functional.interpolate(pic[None], size=(64, 64), mode="bicubic", align_corners=False, antialias=True).clamp(0, 1)
    x = (x - torch.tensor([0.485, 0.456, 0.406])[None, :, None, None]) / torch.tensor([0.229, 0.224, 0.225])[None, :, None, None]
    with torch.no_grad():
        want = hf(pixel_values=x, input_points=torch.tensor([[[[30 * 64 / 80, 30 * 64 / 48]]]]), input_labels=torch.tensor([[[1]]]))
    best = int(want.iou_scores[0, 0].argmax())
    assert abs(float(res.mask_scores[0][1]) - float(want.iou_scores[0, 0, best])) < 1e-3
    ref = torch.sigmoid(torch.nn.functional.interpolate(want.pred_masks[0, :, best][None], size=(48, 80), mode="bilinear",
                                                        align_corners=False))[0, 0]
    assert (res.masks[0][1] - ref).abs().max() < 2e-3
    box = eng.vision.run(ModelSpec(str(d)), VisionRequest(operation="segment", images=[pic], boxes=[[5, 5, 70, 40]]))
    assert box.masks[0].shape == (1, 48, 80)
    with pytest.raises(ValueError):
        eng.vision.run(ModelSpec(str(d)), VisionRequest(operation="segment", images=[pic]))
    with pytest.raises(ValueError):
        eng.vision.run(ModelSpec(str(d)), VisionRequest(operation="embed", images=[pic]))


@pytest.mark.gpu
def test_gpu_bf16_agrees_with_cpu():
    c, hf = _hf(2)
    sd = hf.state_dict()
    cfg = sam2_from_hf(c.to_dict())
    x = torch.randn(1, 3, 64, 64)
    pts, lab = torch.tensor([[[[20.0, 30.0]]]]), torch.tensor([[[1]]])
    m0, i0, _ = Sam2(cfg, "cpu", get=sd.get).segment(x, pts, lab)
    m1, i1, _ = Sam2(cfg, "cuda", get=sd.get).segment(x, pts, lab)          # bf16 on the device
    cos = torch.nn.functional.cosine_similarity(m1.cpu().flatten(), m0.flatten(), dim=0)
    assert cos > 0.98 and (i1.cpu() - i0).abs().max() < 0.05
