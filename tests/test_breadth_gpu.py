"""B200 runs of the breadth models against their CPU statement."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_clip_vision_tower_matches_cpu():
    from hartsyinference_b200.models.encoders.clip_vision import ClipVisionEncoder, tiny_clip_vision
    cfg = tiny_clip_vision()
    cpu = ClipVisionEncoder(cfg, "cpu", seed=4)
    gpu = ClipVisionEncoder(cfg, "cuda", seed=4)
    img = torch.randn(3, cfg.image_size, cfg.image_size, generator=torch.Generator().manual_seed(0))
    a = cpu.hidden_states(img, -2).float()
    b = gpu.hidden_states(img, -2).float().cpu()
    assert torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0) > 0.995
