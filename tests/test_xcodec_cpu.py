"""X-Codec against `transformers.XcodecModel` (tiny random weights): codes from audio and audio from codes."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from hartsyinference_b200.models.audio.xcodec import XCodec  # noqa: E402


def _tiny():
    torch.manual_seed(0)
    dac = transformers.DacConfig(encoder_hidden_size=8, downsampling_ratios=[8, 5, 4, 2], upsampling_ratios=[8, 5, 4, 2],
                                 decoder_hidden_size=64, n_codebooks=2, codebook_size=16, codebook_dim=4, hidden_size=32, sampling_rate=16000)
    hub = transformers.HubertConfig(hidden_size=32, num_hidden_layers=2, num_attention_heads=4, intermediate_size=64, conv_dim=[16] * 7,
                                    num_conv_pos_embeddings=16, num_conv_pos_embedding_groups=4, hidden_dropout=0.0, attention_dropout=0.0,
                                    feat_proj_dropout=0.0, activation_dropout=0.0, layerdrop=0.0, mask_time_prob=0.0)
    cfg = transformers.XcodecConfig(acoustic_model_config=dac, semantic_model_config=hub, codebook_size=32, codebook_dim=64,
                                    target_bandwidths=[0.5, 1.0, 1.5, 2.0])
    model = transformers.XcodecModel(cfg).eval()
    with torch.no_grad():
        for n, b in model.named_buffers():
            if n.endswith("codebook.embed"):
                b.normal_(0, 1.0)
        for n, p in model.named_parameters():
            if n.endswith("alpha"):
                p.uniform_(0.5, 1.5)
    return cfg, model


def test_codes_and_audio_match_transformers():
    cfg, model = _tiny()
    wave = torch.randn(1, 1, 3200) * 0.3
    with torch.no_grad():
        want_codes = model.encode(wave).audio_codes
        want_wave = model.decode(want_codes).audio_values
    mine = XCodec(cfg.to_dict(), model.state_dict().get)
    assert mine.hop == 320 and mine.quantizers == want_codes.shape[1]
    codes = mine.encode(wave)
    assert codes.shape == want_codes.shape and (codes == want_codes).float().mean() > 0.99
    got = mine.decode(want_codes)
    assert got.shape == want_wave[:, 0].shape and torch.allclose(got, want_wave[:, 0], atol=1e-4), float((got - want_wave[:, 0]).abs().max())
    assert torch.equal(mine.encode(wave, quantizers=2), codes[:, :2])
