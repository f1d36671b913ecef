"""Grounding DINO against `transformers.GroundingDinoForObjectDetection` (tiny random weights): phrase masks, text
states, and the final logits / boxes of the whole picture + text model."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from hartsyinference_b200.models.vision.grounding_dino import GroundingDino, GroundingDinoConfig, phrase_masks  # noqa: E402


def _tiny():
    torch.manual_seed(0)
    swin = transformers.SwinConfig(embed_dim=16, depths=[2, 2, 2, 2], num_heads=[2, 2, 4, 4], window_size=4, patch_size=4,
                                   out_features=["stage2", "stage3", "stage4"], hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0,
                                   drop_path_rate=0.0)
    text = transformers.BertConfig(vocab_size=1100, hidden_size=32, num_hidden_layers=2, num_attention_heads=4, intermediate_size=64,
                                   max_position_embeddings=64, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
    cfg = transformers.GroundingDinoConfig(backbone_config=swin, text_config=text, d_model=64, encoder_layers=2, decoder_layers=2,
                                           encoder_attention_heads=4, decoder_attention_heads=4, encoder_ffn_dim=96, decoder_ffn_dim=96,
                                           num_queries=12, max_text_len=32, dropout=0.0, attention_dropout=0.0, activation_dropout=0.0,
                                           fusion_dropout=0.0, fusion_droppath=0.0, text_enhancer_dropout=0.0, disable_custom_kernels=True)
    model = transformers.GroundingDinoForObjectDetection(cfg).eval()
    with torch.no_grad():
        for n, p in model.named_parameters():
            if n.endswith("vision_param") or n.endswith("text_param"):
                p.fill_(0.5)                                  # let the fusion matter
            if "bbox_embed" in n and n.endswith("layers.2.weight"):
                p.normal_(0, 0.05)                            # zero-initialised in the library
    return cfg, model


def test_phrase_masks_follow_the_library():
    from transformers.models.grounding_dino.modeling_grounding_dino import generate_masks_with_special_tokens_and_transfer_map
    ids = torch.tensor([101, 7, 8, 1012, 9, 1012, 10, 11, 12, 1029, 102])
    want_mask, want_pos = generate_masks_with_special_tokens_and_transfer_map(ids[None])
    allowed, pos = phrase_masks(ids)
    assert torch.equal(allowed, want_mask[0]) and torch.equal(pos, want_pos[0])
    assert allowed[1, 2] and not allowed[1, 4] and pos[:3].tolist() == [0, 0, 1] and int(pos[4]) == 0


def test_logits_and_boxes_match_transformers():
    cfg, model = _tiny()
    ids = torch.tensor([[101, 7, 8, 1012, 9, 1012, 10, 11, 1012, 102]])
    pixels = torch.randn(1, 3, 96, 128)
    with torch.no_grad():
        want = model(pixel_values=pixels, input_ids=ids)
    mine = GroundingDino(GroundingDinoConfig.from_hf(cfg.to_dict()), model.state_dict().get)
    text, _, _ = mine.text_states(ids[0])
    logits, boxes = mine.forward(pixels, ids[0])
    assert torch.allclose(boxes, want.pred_boxes[0], atol=2e-4), float((boxes - want.pred_boxes[0]).abs().max())
    got = torch.full((12, 32), float("-inf"))
    got[:, :10] = logits
    finite = torch.isfinite(want.logits[0])
    assert torch.equal(finite, torch.isfinite(got)) and torch.allclose(got[finite], want.logits[0][finite], atol=2e-3)
    found = mine.detect(pixels, ids[0], box_threshold=0.0, text_threshold=0.0)
    assert len(found) == 12 and found[0][1] >= found[-1][1] and len(found[0][2]) == 4


def test_vision_service_detects_with_phrases(tmp_path):
    import json
    from hartsyinference_b200.assets.safetensors import save_file
    from hartsyinference_b200.engine.requests import ModelSpec, VisionRequest
    from hartsyinference_b200.engine.vision_service import VisionService
    cfg, model = _tiny()
    raw = cfg.to_dict()
    raw["model_type"] = "grounding-dino"
    raw["short_side"] = 96
    (tmp_path / "config.json").write_text(json.dumps(raw, default=str))
    save_file({k: v.contiguous() for k, v in model.state_dict().items()}, tmp_path / "model.safetensors")
    vocab = ["[PAD]"] * 1100
    vocab[100], vocab[101], vocab[102], vocab[1012], vocab[1029] = "[UNK]", "[CLS]", "[SEP]", ".", "?"
    for i, wd in enumerate(["a", "cat", "remote", "control", "dog"]):
        vocab[200 + i] = wd
    for i, wd in enumerate(vocab):
        if wd == "[PAD]" and i:
            vocab[i] = f"[unused{i}]"
    (tmp_path / "vocab.txt").write_text("\n".join(vocab) + "\n")
    svc = VisionService("cpu")
    img = (torch.rand(96, 128, 3) * 255).to(torch.uint8)
    res = svc.run(ModelSpec(str(tmp_path)), VisionRequest(operation="detect", images=[img], texts=["a cat", "remote control"],
                                                          score_threshold=0.0, nms_iou=1.0))
    found = res.detections[0]
    assert len(found) == 12 and {d["label"] for d in found} <= {"a cat", "remote control"}
    # the same numbers straight from the model: caption "[CLS] a cat . remote control . [SEP]"
    ids = torch.tensor([101, 200, 201, 1012, 202, 203, 1012, 102])
    mine = GroundingDino(GroundingDinoConfig.from_hf(raw), model.state_dict().get)
    x = img.permute(2, 0, 1).float() / 255
    x = (x - torch.tensor([0.485, 0.456, 0.406])[:, None, None]) / torch.tensor([0.229, 0.224, 0.225])[:, None, None]
    logits, boxes = mine.forward(x[None], ids)
    probs = logits.sigmoid()
    best = torch.maximum(probs[:, 1:3].max(-1)[0], probs[:, 4:6].max(-1)[0]).max()
    assert found[0]["score"] == pytest.approx(float(best), abs=1e-5)
    with pytest.raises(ValueError):
        svc.run(ModelSpec(str(tmp_path)), VisionRequest(operation="detect", images=[img]))
