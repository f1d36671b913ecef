"""Kyutai speech-to-text against `transformers.KyutaiSpeechToTextForConditionalGeneration` (tiny random weights,
greedy): one text token per audio frame, with Mimi codes computed by our codec."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from hartsyinference_b200.models.audio.kyutai_stt import KyutaiStt  # noqa: E402


def _tiny():
    torch.manual_seed(0)
    codec = dict(hidden_size=32, num_filters=4, upsampling_ratios=[4, 3, 2], codebook_size=16, codebook_dim=8,
                 vector_quantization_hidden_dimension=8, num_quantizers=4, num_semantic_quantizers=1, num_hidden_layers=1,
                 num_attention_heads=4, num_key_value_heads=4, head_dim=8, intermediate_size=48, sliding_window=64, upsample_groups=32,
                 sampling_rate=2400, frame_rate=50.0, model_type="mimi")
    cfg = transformers.KyutaiSpeechToTextConfig(codebook_vocab_size=17, vocab_size=41, hidden_size=48, num_hidden_layers=2, num_attention_heads=4,
                                                num_key_value_heads=2, head_dim=12, ffn_dim=128, sliding_window=64, num_codebooks=4,
                                                audio_bos_token_id=16, audio_pad_token_id=41 + 4 * 17, pad_token_id=3, bos_token_id=40,
                                                max_position_embeddings=128, codec_config=codec)
    model = transformers.KyutaiSpeechToTextForConditionalGeneration(cfg).eval()
    with torch.no_grad():
        for name, buf in model.named_buffers():
            if name.endswith("embed_sum"):
                buf.copy_(torch.randn_like(buf))
            elif name.endswith("cluster_usage"):
                buf.copy_(torch.rand_like(buf) + 0.5)
        for m in model.modules():
            if hasattr(m, "_embed"):
                m._embed = None
    return cfg, model


def test_tokens_match_transformers():
    cfg, model = _tiny()
    assert cfg.frame_size == 48
    wave = torch.randn(1, 1, 48 * 20) * 0.3
    with torch.no_grad():
        want = model.generate(input_values=wave, do_sample=False)
    mine = KyutaiStt(cfg.to_dict(), model.state_dict().get)
    got = mine.transcribe_tokens(wave[0, 0])
    assert want.shape[1] == 21 and want[0, 0] == cfg.bos_token_id
    assert got.tolist() == want[0, 1:].tolist()
    padded = mine.transcribe_tokens(wave[0, 0], delay_seconds=0.1, silence_prefix_seconds=0.04)
    assert padded.numel() == (48 * 20 + 96 + int(1.1 * 2400)) // 48
    assert all(t not in (3, 40) for t in mine.text_ids(got))


def test_transcribe_service_hosts_the_checkpoint(tmp_path):
    import json
    from hartsyinference_b200.assets.safetensors import save_file
    from hartsyinference_b200.assets.tokenizer import _bytes_to_unicode
    from hartsyinference_b200.engine.audio_service import TranscribeService
    from hartsyinference_b200.engine.requests import AudioRequest, ModelSpec
    cfg, model = _tiny()
    raw = cfg.to_dict()
    raw["model_type"] = "kyutai_speech_to_text"
    (tmp_path / "config.json").write_text(json.dumps(raw, default=str))
    (tmp_path / "preprocessor_config.json").write_text(json.dumps({"audio_delay_seconds": 0.1, "audio_silence_prefix_seconds": 0.04}))
    save_file({k: v.contiguous() for k, v in model.state_dict().items()}, tmp_path / "model.safetensors")
    b2u = _bytes_to_unicode()
    vocab = {b2u[ord(c)]: 4 + i for i, c in enumerate("abcdefghijklmnopqrstuvwxyz .,!?'-")}
    (tmp_path / "tokenizer.json").write_text(json.dumps({"model": {"type": "BPE", "vocab": vocab, "merges": []}, "added_tokens": [],
                                                         "pre_tokenizer": {"type": "ByteLevel", "add_prefix_space": False}}))
    svc = TranscribeService("cpu")
    wave = torch.randn(4800) * 0.3
    res = svc.run(ModelSpec(str(tmp_path)), AudioRequest(audio=wave, sample_rate=2400))
    mine = KyutaiStt(raw, model.state_dict().get)
    tokens = mine.transcribe_tokens(wave, 0.1, 0.04)
    written = [t for t in tokens.tolist() if t not in (3, 40)]
    assert [t for s in res.segments for t in s.tokens] == written and res.duration_s == pytest.approx(2.0)
    assert all(s.end >= s.start >= 0 for s in res.segments) and svc.loaded_keys() == [f"kyutai:{tmp_path}"]
