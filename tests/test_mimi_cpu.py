"""Mimi codec against `transformers.MimiModel` (tiny random weights): codes from audio, audio from codes, with the
sliding attention window shorter than the clip and a clip length that needs right padding."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from hartsyinference_b200.models.audio.mimi import Mimi, MimiConfig  # noqa: E402


def _tiny(**over):
    kw = dict(hidden_size=32, num_filters=4, upsampling_ratios=[4, 3, 2], codebook_size=16, codebook_dim=8,
              vector_quantization_hidden_dimension=8, num_quantizers=6, num_semantic_quantizers=1, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=4, head_dim=8, intermediate_size=48, sliding_window=5, upsample_groups=32,
              sampling_rate=2400, frame_rate=50.0, layer_scale_initial_scale=0.3)
    kw.update(over)
    torch.manual_seed(0)
    cfg = transformers.MimiConfig(**kw)
    model = transformers.MimiModel(cfg).eval()
    with torch.no_grad():                      # codebooks as a trained model has them: distinct entries, uneven usage
        for name, buf in model.named_buffers():
            if name.endswith("embed_sum"):
                buf.copy_(torch.randn_like(buf))
            elif name.endswith("cluster_usage"):
                buf.copy_(torch.rand_like(buf) + 0.5)
        for m in model.modules():
            if hasattr(m, "_embed"):
                m._embed = None
    return cfg, model


@pytest.mark.parametrize("samples", [960, 1000])
def test_encode_and_decode_match_transformers(samples):
    cfg, model = _tiny()
    assert cfg.encodec_frame_rate == 100.0      # 2400 / 24, halved by the stride-2 stage to the 50 Hz frame rate
    wave = torch.randn(2, 1, samples) * 0.3
    with torch.no_grad():
        want_codes = model.encode(wave).audio_codes
        want_wave = model.decode(want_codes).audio_values
    mine = Mimi(MimiConfig.from_hf(cfg.to_dict()), model.state_dict().get)
    codes = mine.encode(wave)
    assert codes.shape == want_codes.shape and codes.shape[1] == 6 and codes.shape[2] > cfg.sliding_window
    assert (codes == want_codes).float().mean() > 0.99          # a near-tie in a distance may flip an entry
    got = mine.decode(want_codes)
    assert got.shape == want_wave.shape and torch.allclose(got, want_wave, atol=1e-4), float((got - want_wave).abs().max())
    fewer = mine.encode(wave, quantizers=3)
    assert torch.equal(fewer, codes[:, :3])
    assert torch.allclose(mine.decode(want_codes[:, :3]), model.decode(want_codes[:, :3]).audio_values, atol=1e-4)


def test_prefixed_names_and_shortcut_layout():
    cfg, model = _tiny(use_conv_shortcut=True, num_key_value_heads=2)
    wave = torch.randn(1, 1, 720) * 0.3
    with torch.no_grad():
        want = model.decode(model.encode(wave).audio_codes).audio_values
    sd = {"codec_model." + k: v for k, v in model.state_dict().items()}
    mine = Mimi(MimiConfig.from_hf(cfg.to_dict()), sd.get, prefix="codec_model.")
    assert torch.allclose(mine.decode(model.encode(wave).audio_codes), want, atol=1e-4)
    assert mine.cfg.samples_per_frame == 48
