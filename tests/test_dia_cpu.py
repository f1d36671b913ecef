"""Dia against `transformers.DiaForConditionalGeneration` (tiny random weights, greedy): encoder states, decoder logits,
and the generated code matrix with guidance, the top-k filter, the delay pattern and the forced endings."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from hartsyinference_b200.models.audio.dia import Dia  # noqa: E402


def _tiny(seed=3):
    from transformers.models.dia.configuration_dia import DiaDecoderConfig, DiaEncoderConfig
    torch.manual_seed(seed)
    enc = DiaEncoderConfig(max_position_embeddings=64, num_hidden_layers=2, hidden_size=32, num_attention_heads=4, num_key_value_heads=4,
                           head_dim=8, intermediate_size=64, vocab_size=128)
    dec = DiaDecoderConfig(max_position_embeddings=96, num_hidden_layers=2, hidden_size=48, intermediate_size=96, num_attention_heads=4,
                           num_key_value_heads=2, head_dim=12, cross_num_attention_heads=4, cross_head_dim=8, cross_num_key_value_heads=4,
                           cross_hidden_size=32, vocab_size=24, num_channels=4, pad_token_id=21, eos_token_id=20, bos_token_id=22)
    cfg = transformers.DiaConfig(encoder_config=enc, decoder_config=dec, delay_pattern=[0, 2, 3, 5], pad_token_id=21, eos_token_id=20,
                                 bos_token_id=22)
    model = transformers.DiaForConditionalGeneration(cfg).eval()
    with torch.no_grad():                                   # spread the logits so that end ids do come up
        model.logits_dense.weight.mul_(40.0)
    return cfg, model


def test_encoder_and_decoder_match_transformers():
    cfg, model = _tiny()
    mine = Dia(cfg.to_dict(), model.state_dict().get)
    text = torch.tensor([[5, 9, 33, 2, 17, 40]])
    codes = torch.randint(0, 20, (1, 7, 4), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = model(input_ids=text, decoder_input_ids=codes)
    enc = mine.encode_text(text)
    assert torch.allclose(enc, want.encoder_last_hidden_state, atol=1e-5)
    cache = mine.new_cache(enc)
    logits = mine.decode_step(codes, cache)                                  # [1, 7, 4, V]
    assert torch.allclose(logits[0].transpose(0, 1), want.logits, atol=1e-3), float((logits[0].transpose(0, 1) - want.logits).abs().max())
    # stepwise with the cache gives the same as the whole prefix at once
    cache = mine.new_cache(enc)
    steps = torch.cat([mine.decode_step(codes[:, i:i + 1], cache) for i in range(7)], 1)
    assert torch.allclose(steps, logits, atol=1e-4)


@pytest.mark.parametrize("guidance,top_k", [(3.0, 5), (None, None)])
def test_generated_codes_match_transformers(guidance, top_k):
    cfg, model = _tiny()
    mine = Dia(cfg.to_dict(), model.state_dict().get)
    text = torch.tensor([[5, 9, 33, 2, 17, 40, 8]])
    delays, c = cfg.delay_pattern, 4
    # what the processor hands to generate when there is no audio prompt: the start id until each codebook's delay has passed
    prefill = torch.full((1, 1 + max(delays), c), 21)
    for ch, d in enumerate(delays):
        prefill[0, :d + 1, ch] = 22
    kw = dict(input_ids=text, attention_mask=torch.ones_like(text), decoder_input_ids=prefill,
              decoder_attention_mask=torch.ones(1, 1 + max(delays), dtype=torch.long), max_new_tokens=30, do_sample=False)
    if guidance:
        kw.update(guidance_scale=guidance, top_k=top_k)
    with torch.no_grad():
        out = model.generate(**kw)
    seq = out[0]                                                             # [L, C], delayed
    length = seq.shape[0]
    end = length - int((seq[:, 0] == 21).sum()) - 1
    want = torch.stack([seq[(torch.arange(length) + d).clamp(max=length - 1), ch] for ch, d in enumerate(delays)], 1)[1:end].t()
    got = mine.generate_codes(text[0], max_steps=31, guidance=guidance, top_k=top_k)
    assert got.shape == want.shape and got.shape[1] >= 2, (got.shape, want.shape)
    assert torch.equal(got, want)
    assert int(got.max()) < 20                                               # no control id inside the kept frames


def test_audio_needs_the_codec():
    cfg, model = _tiny()
    mine = Dia(cfg.to_dict(), model.state_dict().get)
    with pytest.raises(ValueError):
        mine.generate(torch.tensor([1, 2, 3]))
    with pytest.raises(ValueError):
        mine.encode_text(torch.tensor([[1, 200]]))

    class Codec:
        def decode(self, codes):
            return codes.float().sum(1, keepdim=True).repeat_interleave(4, -1)
    mine.codec = Codec()
    wave = mine.generate(torch.tensor([5, 9, 33, 2, 17, 40, 8]), max_steps=31, guidance=3.0, top_k=5)
    assert wave.numel() == 4 * mine.generate_codes(torch.tensor([5, 9, 33, 2, 17, 40, 8]), max_steps=31, guidance=3.0, top_k=5).shape[1]


def test_speech_service_hosts_a_dia_checkpoint(tmp_path):
    import json
    from hartsyinference_b200.assets.safetensors import save_file
    from hartsyinference_b200.engine.audio_service import SpeechService, _DiaVoice
    from hartsyinference_b200.engine.requests import ModelSpec, SpeechRequest
    from hartsyinference_b200.models.audio.dac import DacCodec, DacConfig
    cfg, model = _tiny()
    raw = cfg.to_dict()
    raw["model_type"] = "dia"
    (tmp_path / "config.json").write_text(json.dumps(raw, default=str))
    save_file({k: v.contiguous() for k, v in model.state_dict().items()}, tmp_path / "model.safetensors")
    dac_cfg = transformers.DacConfig(encoder_hidden_size=8, downsampling_ratios=[2, 4], upsampling_ratios=[4, 2], decoder_hidden_size=32,
                                     n_codebooks=4, codebook_size=32, codebook_dim=4, hidden_size=32, sampling_rate=8000)
    dac = transformers.DacModel(dac_cfg).eval()
    (tmp_path / "dac").mkdir()
    (tmp_path / "dac" / "config.json").write_text(json.dumps(dac_cfg.to_dict(), default=str))
    save_file({k: v.detach().contiguous() for k, v in dac.state_dict().items()}, tmp_path / "dac" / "model.safetensors")
    assert _DiaVoice.text_bytes("[S1] hi [S2] yo") == [1, 32, 104, 105, 32, 2, 32, 121, 111]
    svc = SpeechService("cpu")
    out = svc.run(ModelSpec(str(tmp_path)), SpeechRequest(text="hi", greedy=True, max_seconds=0.02))
    sd = dac.state_dict()
    codec = DacCodec(DacConfig.from_hf(dac_cfg.to_dict()), lambda n: sd.get(n))
    mine = Dia(raw, model.state_dict().get, codec=codec)
    limit = max(2, round(0.02 * 8000 / 8)) + 5 + 2
    want = mine.generate(torch.tensor([1, 32, 104, 105]), max_steps=limit)
    assert out.sample_rate == 8000 and out.samples.numel() == want.numel() > 0
    assert torch.allclose(out.samples, want.clamp(-1, 1), atol=1e-5) and svc.loaded_keys() == [f"dia:{tmp_path}"]
