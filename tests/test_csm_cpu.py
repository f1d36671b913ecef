"""CSM against `transformers.CsmForConditionalGeneration` (tiny random weights, greedy): generated frames and audio,
with a text-only prompt and with context audio in the prompt."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from hartsyinference_b200.models.audio.csm import Csm  # noqa: E402


def _tiny(rope=None):
    torch.manual_seed(0)
    codec = dict(hidden_size=32, num_filters=4, upsampling_ratios=[4, 3, 2], codebook_size=32, codebook_dim=8,
                 vector_quantization_hidden_dimension=8, num_quantizers=4, num_semantic_quantizers=1, num_hidden_layers=1,
                 num_attention_heads=4, num_key_value_heads=4, head_dim=8, intermediate_size=48, sliding_window=6, upsample_groups=32,
                 sampling_rate=2400, frame_rate=50.0, model_type="mimi")
    depth = dict(num_codebooks=4, backbone_hidden_size=48, vocab_size=35, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                 num_attention_heads=4, num_key_value_heads=2, head_dim=8, max_position_embeddings=5)
    kw = dict(num_codebooks=4, vocab_size=35, text_vocab_size=40, hidden_size=48, intermediate_size=96, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=2, head_dim=12, max_position_embeddings=256, pad_token_id=37,
              codebook_pad_token_id=34, codebook_eos_token_id=0, bos_token_id=1, audio_token_id=37, audio_eos_token_id=38,
              depth_decoder_config=depth, codec_config=codec)
    if rope:
        kw["rope_parameters"] = rope
        depth["rope_parameters"] = rope
    cfg = transformers.CsmConfig(**kw)
    model = transformers.CsmForConditionalGeneration(cfg).eval()
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


@pytest.mark.parametrize("rope", [None, {"rope_type": "llama3", "rope_theta": 10000.0, "factor": 8.0, "low_freq_factor": 1.0,
                                          "high_freq_factor": 4.0, "original_max_position_embeddings": 16}])
def test_generated_frames_and_audio_match_transformers(rope):
    cfg, model = _tiny(rope)
    ids = torch.tensor([[1, 5, 9, 22, 7, 3]])
    with torch.no_grad():
        want = model.generate(input_ids=ids, max_new_tokens=7, do_sample=False, depth_decoder_do_sample=False)
        want_audio = model.generate(input_ids=ids, max_new_tokens=7, do_sample=False, depth_decoder_do_sample=False, output_audio=True)
    mine = Csm(cfg.to_dict(), model.state_dict().get)
    frames = mine.generate_codes(ids[0], max_frames=7)
    n = frames.shape[0]
    assert n >= 3 and torch.equal(frames, want[0][:n])
    if n < want.shape[1]:                                   # theirs goes on after the closing frame; ours stops there
        assert bool((want[0][n] == 0).all())
    wave = mine.generate(ids[0], max_frames=7)
    assert wave.shape == want_audio[0].shape and torch.allclose(wave, want_audio[0], atol=1e-4)


def test_context_audio_in_the_prompt():
    cfg, model = _tiny()
    wave = torch.randn(1, 480) * 0.3                         # 10 frames of 48 samples
    ids = torch.tensor([[1, 5, 9] + [37] * 10 + [38, 1, 6, 4]])
    cut = torch.tensor([[480]])
    with torch.no_grad():
        # the audio placeholder doubles as the padding id, so the mask has to be given (the processor does)
        want = model.generate(input_ids=ids, input_values=wave[None], input_values_cutoffs=cut, attention_mask=torch.ones_like(ids),
                              max_new_tokens=5, do_sample=False, depth_decoder_do_sample=False)
    mine = Csm(cfg.to_dict(), model.state_dict().get)
    frames = mine.generate_codes(ids[0], [wave[0]], max_frames=5)
    assert frames.shape[0] >= 2 and torch.equal(frames, want[0][:frames.shape[0]])
    with pytest.raises(ValueError):
        mine.generate_codes(ids[0], None, max_frames=2)
    with pytest.raises(ValueError):
        mine.generate_codes(ids[0], [wave[0, :240]], max_frames=2)
    again = mine.generate_codes(ids[0], [wave[0]], max_frames=5, sample=True, seed=4)
    assert torch.equal(again, mine.generate_codes(ids[0], [wave[0]], max_frames=5, sample=True, seed=4))


def test_speech_service_hosts_a_csm_checkpoint(tmp_path):
    import json
    from hartsyinference_b200.assets.safetensors import save_file
    from hartsyinference_b200.assets.tokenizer import _bytes_to_unicode
    from hartsyinference_b200.engine.audio_service import SpeechService
    from hartsyinference_b200.engine.requests import ModelSpec, SpeechRequest
    cfg, model = _tiny()
    raw = cfg.to_dict()
    raw["model_type"] = "csm"
    raw["text_vocab_size"] = 40
    (tmp_path / "config.json").write_text(json.dumps(raw, default=str))
    sd = {k: v.contiguous() for k, v in model.state_dict().items()}
    save_file(sd, tmp_path / "model.safetensors")
    b2u = _bytes_to_unicode()
    chars = "[]0123456789 abcdefghijklmnopqrstu"
    vocab = {b2u[ord(c)]: 2 + i for i, c in enumerate(chars)}
    (tmp_path / "tokenizer.json").write_text(json.dumps({
        "model": {"type": "BPE", "vocab": vocab, "merges": []},
        "added_tokens": [{"id": 1, "content": "<|begin_of_text|>", "special": True}, {"id": 39, "content": "<|end_of_text|>", "special": True}],
        "pre_tokenizer": {"type": "ByteLevel", "add_prefix_space": False}}))
    svc = SpeechService("cpu")
    out = svc.run(ModelSpec(str(tmp_path)), SpeechRequest(text="hello", voice="1", greedy=True, max_seconds=0.2))
    ids = [1] + [vocab[b2u[ord(c)]] for c in "[1]hello"] + [39]
    want = Csm(raw, model.state_dict().get).generate(torch.tensor(ids), max_frames=10)
    assert out.sample_rate == 2400 and out.samples.shape == want.shape and torch.allclose(out.samples, want.clamp(-1, 1), atol=1e-5)
    assert svc.loaded_keys() == [f"csm:{tmp_path}"]
