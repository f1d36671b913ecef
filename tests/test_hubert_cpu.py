"""HuBERT / wav2vec 2.0 encoder against `transformers` (tiny random weights): both normalisation layouts, the
intermediate layers downstream models read, and the wav2vec 2.0 checkpoint names."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from hartsyinference_b200.models.audio.hubert import Hubert, HubertConfig  # noqa: E402


def _cfg(kind, stable, norm):
    kw = dict(hidden_size=32, num_hidden_layers=3, num_attention_heads=4, intermediate_size=64, conv_dim=[16] * 7,
              num_conv_pos_embeddings=16, num_conv_pos_embedding_groups=4, do_stable_layer_norm=stable, feat_extract_norm=norm,
              conv_bias=norm == "layer", vocab_size=32, hidden_dropout=0.0, attention_dropout=0.0, feat_proj_dropout=0.0,
              activation_dropout=0.0, layerdrop=0.0, mask_time_prob=0.0)
    return (transformers.HubertConfig if kind == "hubert" else transformers.Wav2Vec2Config)(**kw)


@pytest.mark.parametrize("kind,stable,norm", [("hubert", False, "group"), ("hubert", True, "layer"), ("wav2vec2", False, "group")])
def test_hidden_states_match_transformers(kind, stable, norm):
    torch.manual_seed(0)
    hf_cfg = _cfg(kind, stable, norm)
    model = (transformers.HubertModel if kind == "hubert" else transformers.Wav2Vec2Model)(hf_cfg).eval()
    wave = torch.randn(2, 4000)
    with torch.no_grad():
        want = model(wave, output_hidden_states=True)
    sd = model.state_dict()
    mine = Hubert(HubertConfig.from_hf(hf_cfg.to_dict()), sd.get)
    x = wave
    if norm == "layer":                       # the released large models expect a normalised waveform; so does ours
        x = (wave - wave.mean(-1, keepdim=True)) / torch.sqrt(wave.var(-1, keepdim=True, unbiased=False) + 1e-7)
        with torch.no_grad():
            want = model(x, output_hidden_states=True)
    got = mine(wave)
    assert got.shape == want.last_hidden_state.shape == (2, mine.frames(4000), 32)
    assert torch.allclose(got, want.last_hidden_state, atol=2e-4), float((got - want.last_hidden_state).abs().max())
    mid = mine.hidden_states(wave, layer=2)
    assert torch.allclose(mid, want.hidden_states[2], atol=2e-4)
    # prefixed names (a checkpoint saved from a model with a head) load too
    prefixed = {("hubert." if kind == "hubert" else "wav2vec2.") + k: v for k, v in sd.items()}
    assert torch.equal(Hubert(HubertConfig.from_hf(hf_cfg.to_dict()), prefixed.get)(wave), got)
