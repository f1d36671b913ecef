"""RT-DETR (models/vision/rtdetr.py) against ``transformers.RTDetrForObjectDetection`` with random tiny
weights, the deformable-attention op against the transformers module's own statement, and the CUDA
kernel against the fp32 reference."""
import pytest
import torch

from hartsyinference_b200 import ops
from hartsyinference_b200.models.vision.rtdetr import RtDetr, rtdetr_from_hf
from hartsyinference_b200.ops import reference as R


def _hf(layer_type, seed):
    from transformers import RTDetrConfig, RTDetrForObjectDetection, RTDetrResNetConfig
    torch.manual_seed(seed)
    bottleneck = layer_type == "bottleneck"
    bc = RTDetrResNetConfig(embedding_size=16, hidden_sizes=[32, 48, 64, 96] if bottleneck else [16, 32, 48, 64],
                            depths=[2, 1, 2, 1], layer_type=layer_type, out_features=["stage2", "stage3", "stage4"])
    cfg = RTDetrConfig(backbone_config=bc, encoder_hidden_dim=32, encoder_in_channels=[48, 64, 96] if bottleneck else [32, 48, 64],
                       d_model=32, encoder_ffn_dim=64, decoder_ffn_dim=64, encoder_attention_heads=4, decoder_attention_heads=4,
                       decoder_layers=3, num_queries=12, num_labels=5, decoder_in_channels=[32, 32, 32], num_denoising=0,
                       anchor_image_size=None, hidden_expansion=0.5 if bottleneck else 1.0)
    m = RTDetrForObjectDetection(cfg).eval()
    with torch.no_grad():                      # random batch-norm statistics, so that the folding is exercised
        for n, b in m.named_buffers():
            if n.endswith("running_mean"):
                b.normal_(0, 0.2)
            elif n.endswith("running_var"):
                b.uniform_(0.5, 1.5)
        for n, p in m.named_parameters():
            if "norm" in n and n.endswith("bias"):
                p.normal_(0, 0.1)
    return cfg, m


@pytest.mark.parametrize("layer_type", ["basic", "bottleneck"])
def test_matches_transformers(layer_type):
    cfg, m = _hf(layer_type, 3)
    sd = m.state_dict()
    mine = RtDetr(rtdetr_from_hf(cfg.to_dict()), "cpu", get=sd.get)
    assert mine.cfg.out_stages == (1, 2, 3) and mine.cfg.layer_type == layer_type
    x = torch.rand(2, 3, 64, 96)
    with torch.no_grad():
        want = m(pixel_values=x)
    logits, boxes = mine.forward(x)
    assert logits.shape == want.logits.shape and boxes.shape == want.pred_boxes.shape
    assert (logits - want.logits).abs().max() < 2e-4, (logits - want.logits).abs().max()
    assert (boxes - want.pred_boxes).abs().max() < 2e-4
    found = mine.detect(x, threshold=0.0)
    assert len(found) == 2 and len(found[0]) == 12 and found[0][0][1] >= found[0][-1][1]


def test_msda_reference_matches_transformers_module():
    from transformers.models.rt_detr.modeling_rt_detr import MultiScaleDeformableAttention
    torch.manual_seed(0)
    b, q, heads, d, lv, pts = 2, 7, 4, 8, 3, 4
    shapes = [(8, 10), (4, 5), (2, 3)]
    value = torch.randn(b, sum(h * w for h, w in shapes), heads, d)
    off = torch.randn(b, q, heads, lv, pts, 2) * 2
    logits = torch.randn(b, q, heads, lv, pts)
    ref = torch.rand(b, q, 4) * 0.8 + 0.1
    w = torch.softmax(logits.reshape(b, q, heads, -1), -1).reshape(b, q, heads, lv, pts)
    loc = ref[:, :, None, None, None, :2] + off / pts * ref[:, :, None, None, None, 2:] * 0.5
    want = MultiScaleDeformableAttention()(value, torch.tensor(shapes), shapes, None, loc, w, 64)
    assert (ops.msda(value, shapes, off, logits, ref) - want).abs().max() < 1e-5
    ref2 = torch.rand(b, q, lv, 2)                      # per-level points (the encoder form of Deformable DETR)
    norm = torch.tensor([[w_, h_] for h_, w_ in shapes], dtype=torch.float32)
    loc2 = ref2[:, :, None, :, None, :] + off / norm[None, None, None, :, None, :]
    want2 = MultiScaleDeformableAttention()(value, torch.tensor(shapes), shapes, None, loc2, w, 64)
    assert (ops.msda(value, shapes, off, logits, ref2) - want2).abs().max() < 1e-5


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,d,lv,pts,ref_dim", [(8, 32, 3, 4, 4), (4, 64, 4, 8, 2), (2, 128, 1, 3, 4), (3, 24, 2, 16, 2)])
def test_msda_kernel_matches_reference(dtype, heads, d, lv, pts, ref_dim):
    torch.manual_seed(1)
    dev = "cuda"
    shapes = [(80, 80), (40, 40), (20, 20), (10, 13)][:lv]
    b, q = 2, 300
    value = torch.randn(b, sum(h * w for h, w in shapes), heads, d, device=dev).to(dtype)
    off = torch.randn(b, q, heads, lv, pts, 2, device=dev) * 3
    logits = torch.randn(b, q, heads, lv, pts, device=dev) * 2
    # references near and across the borders, so that corners fall outside the maps
    ref = (torch.rand(b, q, lv, 2, device=dev) * 1.2 - 0.1) if ref_dim == 2 else \
        torch.cat([torch.rand(b, q, 2, device=dev) * 1.2 - 0.1, torch.rand(b, q, 2, device=dev) * 0.6], -1)
    got = ops.msda(value, shapes, off, logits, ref)
    want = R.msda(value.float(), shapes, off, logits, ref)
    assert got.dtype == dtype
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    assert (got.float() - want).abs().max() < tol * max(1.0, float(want.abs().max()))


@pytest.mark.gpu
def test_gpu_model_matches_cpu_model():
    cfg, m = _hf("bottleneck", 5)
    sd = m.state_dict()
    c = rtdetr_from_hf(cfg.to_dict())
    x = torch.rand(1, 3, 64, 64)
    cpu, gpu = RtDetr(c, "cpu", get=sd.get), RtDetr(c, "cuda", get=sd.get, dtype=torch.float32)
    tf32 = torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32
    torch.backends.cudnn.allow_tf32 = torch.backends.cuda.matmul.allow_tf32 = False
    try:
        for a, b in zip(cpu.encoder(cpu.backbone(x)), gpu.encoder(gpu.backbone(x.cuda()))):
            assert (b.cpu() - a).abs().max() < 1e-3 * max(1.0, float(a.abs().max()))
        l0, b0 = cpu.forward(x)
        l1, b1 = gpu.forward(x)
    finally:
        torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32 = tf32
    # random weights put many proposals on near-ties, so the selected query sets may differ in a few
    # places: every GPU query that has a CPU twin (same box) must carry the same class scores
    d = (b1.cpu()[0][:, None] - b0[0][None]).abs().amax(-1)            # [Q gpu, Q cpu]
    near, idx = d.min(1)
    twins = near < 1e-3
    assert int(twins.sum()) >= 9, near
    assert (l1.cpu()[0][twins] - l0[0][idx[twins]]).abs().max() < 5e-3


def test_vision_service_detects_with_a_closed_label_set(tmp_path):
    from hartsyinference_b200.assets.safetensors import save_file
    from hartsyinference_b200.engine import InferenceEngine
    from hartsyinference_b200.engine.requests import ModelSpec, VisionRequest
    import json
    cfg, m = _hf("basic", 7)
    d = cfg.to_dict()
    d["id2label"] = {str(i): n for i, n in enumerate(["cat", "dog", "car", "tree", "cup"])}
    d["anchor_image_size"] = [64, 64]
    (tmp_path / "det").mkdir()
    (tmp_path / "det" / "config.json").write_text(json.dumps(d))
    save_file({k: v.contiguous() for k, v in m.state_dict().items() if "num_batches_tracked" not in k},
              tmp_path / "det" / "model.safetensors")
    pic = torch.rand(3, 50, 70)
    eng = InferenceEngine("cpu")
    res = eng.vision.run(ModelSpec(str(tmp_path / "det")), VisionRequest(operation="detect", images=[pic], score_threshold=0.0))
    found = res.detections[0]
    assert len(found) == 12 and {f["label"] for f in found} <= {"cat", "dog", "car", "tree", "cup"}
    assert all(f["score"] >= g["score"] for f, g in zip(found, found[1:]))
    with torch.no_grad():                       # the best box against transformers on the same squeezed picture
        x = torch.nn.functional.interpolate(pic[None], size=(64, 64), mode="bicubic", align_corners=False, antialias=True).clamp(0, 1)
        out = m(pixel_values=x)
    s = torch.sigmoid(out.logits[0]).flatten()
    i = int(s.argmax())
    cx, cy, bw, bh = out.pred_boxes[0, i // 5].tolist()
    assert abs(found[0]["score"] - float(s[i])) < 1e-3
    want = [(cx - bw / 2) * 70, (cy - bh / 2) * 50, (cx + bw / 2) * 70, (cy + bh / 2) * 50]
    assert max(abs(a - b) for a, b in zip(found[0]["box"], want)) < 0.05
    only = eng.vision.run(ModelSpec(str(tmp_path / "det")),
                          VisionRequest(operation="detect", images=[pic], texts=[found[0]["label"].upper()],
                                        score_threshold=0.0)).detections[0]
    assert only and all(f["label"] == found[0]["label"] for f in only)
