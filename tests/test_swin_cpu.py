"""Swin backbone against `transformers.SwinBackbone` (tiny random weights): shifted windows, padding to the window size,
odd map sizes at the merges, per-stage output norms."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from hartsyinference_b200.models.encoders.swin import SwinBackbone, SwinConfig  # noqa: E402


@pytest.mark.parametrize("size", [(64, 64), (75, 98)])
def test_feature_maps_match_transformers(size):
    torch.manual_seed(0)
    cfg = transformers.SwinConfig(embed_dim=16, depths=[2, 2, 2, 2], num_heads=[2, 2, 4, 4], window_size=4, patch_size=4,
                                  out_features=["stage2", "stage3", "stage4"], hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0,
                                  drop_path_rate=0.0)
    model = transformers.SwinBackbone(cfg).eval()
    with torch.no_grad():
        for n, p in model.named_parameters():
            if n.endswith("relative_position_bias_table"):
                p.normal_(0, 0.5)
    x = torch.randn(2, 3, *size)
    with torch.no_grad():
        want = model(x).feature_maps
    mine = SwinBackbone(SwinConfig.from_hf(cfg.to_dict()), model.state_dict().get)
    got = mine(x)
    assert len(got) == 3 and mine.cfg.out_stages == (2, 3, 4)
    for a, b in zip(got, want):
        assert a.shape == b.shape and torch.allclose(a, b, atol=2e-4), float((a - b).abs().max())
