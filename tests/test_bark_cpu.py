"""Bark against `transformers.BarkModel` (tiny random weights, greedy decoding): the three token stages, with and
without a voice prompt, several coarse windows and several fine windows, the EnCodec decode, and the speech service."""
import json

import numpy as np
import pytest
import torch

transformers = pytest.importorskip("transformers")

from hartsyinference_b200.models.audio.bark import Bark  # noqa: E402

CODEBOOK = 16


def _tiny():
    from transformers import BarkConfig, BarkModel, EncodecConfig
    from transformers.models.bark.configuration_bark import BarkCoarseConfig, BarkFineConfig, BarkSemanticConfig
    from transformers.models.bark.generation_configuration_bark import (BarkCoarseGenerationConfig, BarkFineGenerationConfig,
                                                                        BarkSemanticGenerationConfig)
    torch.manual_seed(0)
    kw = dict(hidden_size=32, num_layers=2, num_heads=2)
    sem = BarkSemanticConfig(block_size=128, input_vocab_size=60, output_vocab_size=60, bias=False, **kw)
    co = BarkCoarseConfig(block_size=128, input_vocab_size=66, output_vocab_size=66, bias=True, **kw)
    fi = BarkFineConfig(block_size=64, input_vocab_size=CODEBOOK + 1, output_vocab_size=CODEBOOK + 1, n_codes_total=8, n_codes_given=1, **kw)
    codec = EncodecConfig(hidden_size=16, num_filters=4, codebook_size=CODEBOOK, codebook_dim=16, upsampling_ratios=[4, 2],
                          target_bandwidths=[96.0], sampling_rate=24000)
    cfg = BarkConfig(semantic_config=sem.to_dict(), coarse_acoustics_config=co.to_dict(), fine_acoustics_config=fi.to_dict(),
                     codec_config=codec.to_dict())
    model = BarkModel(cfg).eval()
    sg = BarkSemanticGenerationConfig(eos_token_id=30, text_encoding_offset=40, text_pad_token=58, semantic_infer_token=59,
                                      semantic_vocab_size=30, max_input_semantic_length=8, semantic_rate_hz=49.9, min_eos_p=None,
                                      max_new_tokens=24, do_sample=False, renormalize_logits=True)
    cg = BarkCoarseGenerationConfig(coarse_semantic_pad_token=62, coarse_rate_hz=75, n_coarse_codebooks=2, coarse_infer_token=64,
                                    max_coarse_input_length=8, max_coarse_history=20, sliding_window_len=6, do_sample=False,
                                    renormalize_logits=True, max_new_tokens=None)
    fg = BarkFineGenerationConfig(n_fine_codebooks=8, max_fine_history_length=8, max_fine_input_length=16)
    return cfg, model, sg, cg, fg


def _theirs(model, sg, cg, fg, text, history):
    ids = torch.zeros(1, 8, dtype=torch.long)
    ids[0, :len(text)] = torch.tensor(text)
    mask = (torch.arange(8) < len(text)).long()[None]
    with torch.no_grad():
        s = model.semantic.generate(ids, semantic_generation_config=sg, attention_mask=mask, history_prompt=history)
        c = model.coarse_acoustics.generate(s.clone(), semantic_generation_config=sg, coarse_generation_config=cg,
                                            codebook_size=CODEBOOK, history_prompt=history)
        f = model.fine_acoustics.generate(c, semantic_generation_config=sg, coarse_generation_config=cg, fine_generation_config=fg,
                                          codebook_size=CODEBOOK, history_prompt=history)
        wav = model.codec_decode(f)
    return s[0], c[0], f[0], wav[0]


def _mine(cfg, model, sg, cg, fg):
    gen = {"semantic_config": sg.to_dict(), "coarse_acoustics_config": cg.to_dict(), "fine_acoustics_config": fg.to_dict(),
           "codebook_size": CODEBOOK}
    return Bark(cfg.to_dict(), model.state_dict().get, "cpu", generation=gen), gen


@pytest.mark.parametrize("with_voice", [False, True])
def test_three_stages_and_codec_match_transformers(with_voice):
    cfg, model, sg, cg, fg = _tiny()
    history = None
    if with_voice:
        g = torch.Generator().manual_seed(5)
        history = {"semantic_prompt": torch.randint(0, 30, (12,), generator=g),
                   "coarse_prompt": torch.randint(0, CODEBOOK, (2, 18), generator=g),
                   "fine_prompt": torch.randint(0, CODEBOOK, (8, 18), generator=g)}
    text = [3, 7, 1, 12, 5]
    s, c, f, wav = _theirs(model, sg, cg, fg, text, history)
    bark, _ = _mine(cfg, model, sg, cg, fg)
    my_s = bark.semantic_tokens(torch.tensor(text), history, sample=False)
    n = int((s != 30).sum())
    assert my_s.tolist() == s[:n].tolist() and n > 4
    my_c = bark.coarse_tokens(my_s, history, sample=False)
    assert my_c.tolist() == c.tolist() and my_c.numel() > 2 * cg.sliding_window_len          # several windows
    my_f = bark.fine_codes(my_c, history)
    assert torch.equal(my_f, f.long())
    if with_voice:
        assert my_f.shape[1] + fg.max_fine_history_length > fg.max_fine_input_length          # several fine windows
    my_wav = bark.generate(torch.tensor(text), history, sample=False)
    assert my_wav.shape == wav.shape and torch.allclose(my_wav, wav, atol=1e-5)


def test_end_token_priority_and_sampling_are_reproducible():
    cfg, model, sg, cg, fg = _tiny()
    bark, _ = _mine(cfg, model, sg, cg, fg)
    text = torch.tensor([3, 7, 1, 12, 5])
    a = bark.semantic_tokens(text, sample=True, seed=3)
    b = bark.semantic_tokens(text, sample=True, seed=3)
    assert a.tolist() == b.tolist() and all(t < 30 for t in a.tolist())
    bark.gen.min_eos_p = 1e-6                  # any end-token mass at all now ends the utterance at once
    assert bark.semantic_tokens(text, sample=False).numel() == 0
    assert bark.generate(text, sample=False).numel() == 0


def test_speech_service_hosts_a_bark_checkpoint(tmp_path):
    from hartsyinference_b200.assets.safetensors import save_file
    from hartsyinference_b200.engine.audio_service import SpeechService
    from hartsyinference_b200.engine.requests import ModelSpec, SpeechRequest
    cfg, model, sg, cg, fg = _tiny()
    bark, gen = _mine(cfg, model, sg, cg, fg)
    raw = cfg.to_dict()
    raw["model_type"] = "bark"
    (tmp_path / "config.json").write_text(json.dumps(raw, default=str))
    (tmp_path / "generation_config.json").write_text(json.dumps(gen, default=str))
    save_file({k: v.contiguous() for k, v in model.state_dict().items() if not k.endswith("attn.bias")}, tmp_path / "model.safetensors")
    vocab = ["[PAD]", "[UNK]", "[CLS]", "[SEP]", "hello", "there", "general", "##s", ",", "!", "a", "b", "c", "d", "e", "f"]
    (tmp_path / "vocab.txt").write_text("\n".join(vocab) + "\n")
    voices = tmp_path / "speaker_embeddings"
    voices.mkdir()
    g = torch.Generator().manual_seed(9)
    np.save(voices / "v2_semantic_prompt.npy", torch.randint(0, 30, (10,), generator=g).numpy())
    np.save(voices / "v2_coarse_prompt.npy", torch.randint(0, CODEBOOK, (2, 15), generator=g).numpy())
    np.save(voices / "v2_fine_prompt.npy", torch.randint(0, CODEBOOK, (8, 15), generator=g).numpy())
    svc = SpeechService("cpu")
    spec = ModelSpec(str(tmp_path))
    out = svc.run(spec, SpeechRequest(text="Hello there, generals!", greedy=True))
    ids = torch.tensor([4, 5, 8, 6, 7, 9])
    want = bark.generate(ids, sample=False)
    assert out.sample_rate == 24000 and out.samples.shape == want.shape and torch.allclose(out.samples, want.clamp(-1, 1), atol=1e-5)
    voiced = svc.run(spec, SpeechRequest(text="Hello there", voice="v2", greedy=True))
    assert voiced.samples.numel() > 0 and svc.loaded_keys() == [f"bark:{tmp_path}"]
    with pytest.raises(ValueError):
        svc.run(spec, SpeechRequest(text="Hello", voice="nobody"))
