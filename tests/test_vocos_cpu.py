"""Vocos: structure pinned by the parameter count of the released mel model, the block arithmetic by a restatement,
the inversion by a round trip through torch's STFT."""
import torch
import torch.nn.functional as F

from hartsyinference_b200.models.audio.vocos import Vocos, VocosConfig


def test_released_model_structure():
    v = Vocos(VocosConfig(), device="meta")
    spec = v.spectrum(torch.empty(1, 100, 12, device="meta"))
    assert spec.shape == (1, 513, 12)
    assert sum(t.numel() for t in v._w.values()) == 13_531_650
    assert v._w["backbone.convnext.7.pwconv1.weight"].shape == (1536, 512) and v._w["head.out.weight"].shape == (1026, 512)
    cfg = VocosConfig.from_dict({"backbone": {"init_args": {"input_channels": 80, "dim": 384, "intermediate_dim": 1152, "num_layers": 4}},
                                 "head": {"init_args": {"n_fft": 512, "hop_length": 128}},
                                 "feature_extractor": {"init_args": {"sample_rate": 16000}}})
    assert (cfg.in_channels, cfg.dim, cfg.layers, cfg.n_fft, cfg.hop, cfg.sampling_rate) == (80, 384, 4, 512, 128, 16000)


def test_block_arithmetic_and_inversion():
    cfg = VocosConfig(in_channels=6, dim=8, intermediate=24, layers=1, n_fft=64, hop=16)
    v = Vocos(cfg, seed=1)
    x = torch.randn(2, 6, 20)
    spec = v.spectrum(x)
    w = v._w
    h = F.conv1d(x, w["backbone.embed.weight"], w["backbone.embed.bias"], padding=3)
    h = F.layer_norm(h.transpose(1, 2), (8,), w["backbone.norm.weight"], w["backbone.norm.bias"], 1e-6).transpose(1, 2)
    y = F.conv1d(h, w["backbone.convnext.0.dwconv.weight"], w["backbone.convnext.0.dwconv.bias"], padding=3, groups=8).transpose(1, 2)
    y = F.layer_norm(y, (8,), w["backbone.convnext.0.norm.weight"], w["backbone.convnext.0.norm.bias"], 1e-6)
    y = F.linear(F.gelu(F.linear(y, w["backbone.convnext.0.pwconv1.weight"], w["backbone.convnext.0.pwconv1.bias"])),
                 w["backbone.convnext.0.pwconv2.weight"], w["backbone.convnext.0.pwconv2.bias"]) * w["backbone.convnext.0.gamma"]
    h = F.layer_norm((h + y.transpose(1, 2)).transpose(1, 2), (8,), w["backbone.final_layer_norm.weight"], w["backbone.final_layer_norm.bias"], 1e-6)
    out = F.linear(h, w["head.out.weight"], w["head.out.bias"]).transpose(1, 2)
    mag, ph = out.chunk(2, 1)
    want = torch.complex(mag.exp().clamp(max=100) * ph.cos(), mag.exp().clamp(max=100) * ph.sin())
    assert spec.shape == (2, 33, 20) and torch.allclose(spec, want, atol=1e-5)
    # a spectrum that came from audio is inverted to that audio
    audio = torch.randn(1, 16 * 30)
    s = torch.stft(audio, 64, 16, 64, torch.hann_window(64), center=True, return_complex=True)
    back = torch.istft(s, 64, 16, 64, torch.hann_window(64), center=True)
    assert torch.allclose(back, audio[:, :back.shape[1]], atol=1e-5)
    assert v(x).shape == (2, 19 * 16)
