"""Audio front end and Whisper: features against transformers' extractor, model parity against
transformers' WhisperForConditionalGeneration, decoding grammar, windowing."""
import math

import pytest
import torch

from hartsyinference_b200.audio import log_mel_spectrogram, mel_filterbank, read_wav, resample, write_wav
from hartsyinference_b200.models.audio import WhisperModel, tiny_whisper
from hartsyinference_b200.pipelines.whisper import (WhisperOptions, WhisperPipeline, WhisperVocab)


def test_wav_roundtrip_and_formats():
    x = torch.sin(torch.arange(4000) * 0.05)[None].repeat(2, 1) * torch.tensor([[0.5], [-0.25]])
    y, r = read_wav(write_wav(None, x, 22050))
    assert r == 22050 and y.shape == x.shape and (y - x).abs().max() < 1e-4
    y, r = read_wav(write_wav(None, x[0], 8000, float32=True))
    assert r == 8000 and torch.equal(y[0], x[0])
    with pytest.raises(ValueError):
        read_wav(b"RIFFxxxxWAVE")
    with pytest.raises(ValueError):
        read_wav(b"nope")


def test_resample_keeps_a_tone():
    t = torch.arange(48000) / 48000.0
    s = torch.sin(2 * math.pi * 440 * t)
    d = resample(s, 48000, 16000)
    ref = torch.sin(2 * math.pi * 440 * torch.arange(16000) / 16000.0)
    assert d.shape == ref.shape and (d[200:-200] - ref[200:-200]).abs().max() < 2e-3
    u = resample(d, 16000, 44100)
    ref = torch.sin(2 * math.pi * 440 * torch.arange(44100) / 44100.0)
    assert u.shape == ref.shape and (u[500:-500] - ref[500:-500]).abs().max() < 2e-3
    # content above the new Nyquist is removed, not aliased
    hi = torch.sin(2 * math.pi * 11000 * t)
    assert resample(hi, 48000, 16000)[200:-200].abs().max() < 0.02


def test_log_mel_matches_transformers_extractor():
    tr = pytest.importorskip("transformers")
    x = torch.randn(16000 * 3, generator=torch.Generator().manual_seed(0)) * 0.1
    for mels in (80, 128):
        fe = tr.WhisperFeatureExtractor(feature_size=mels)
        ref = fe(x.numpy(), sampling_rate=16000, return_tensors="pt").input_features[0]
        mine = log_mel_spectrogram(x, n_mels=mels)
        assert mine.shape == ref.shape == (mels, 3000) and (mine - ref).abs().max() < 1e-4
    fb = mel_filterbank(40, 512, 16000, htk=True, norm_slaney=False)
    assert fb.shape == (40, 257) and fb.max() <= 1.0 + 1e-6 and (fb.sum(1) > 0).all()


def _hf_pair():
    tr = pytest.importorskip("transformers")
    cfg = tiny_whisper()
    hc = tr.WhisperConfig(vocab_size=cfg.vocab, num_mel_bins=cfg.n_mels, d_model=cfg.width, encoder_layers=cfg.enc_layers,
                          decoder_layers=cfg.dec_layers, encoder_attention_heads=cfg.heads, decoder_attention_heads=cfg.heads,
                          encoder_ffn_dim=cfg.ffn, decoder_ffn_dim=cfg.ffn, max_source_positions=cfg.max_source,
                          max_target_positions=cfg.max_target, pad_token_id=0, bos_token_id=1, eos_token_id=2,
                          decoder_start_token_id=3, suppress_tokens=None, begin_suppress_tokens=None)
    torch.manual_seed(0)
    hf = tr.WhisperForConditionalGeneration(hc).eval()
    sd = {k: v.detach() for k, v in hf.state_dict().items()}
    return cfg, hf, WhisperModel(cfg, "cpu", get=lambda n: sd.get(n))


def test_whisper_matches_transformers():
    cfg, hf, m = _hf_pair()
    mel = torch.randn(cfg.n_mels, 2 * cfg.max_source, generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        enc_ref = hf.model.encoder(mel[None]).last_hidden_state[0]
    enc = m.encode(mel)
    assert torch.nn.functional.cosine_similarity(enc.float().flatten(), enc_ref.flatten(), dim=0) > 0.999
    toks = torch.tensor([3, 10, 20, 30, 40, 50])
    with torch.no_grad():
        ref = hf(input_features=mel[None], decoder_input_ids=toks[None]).logits[0]
    st = m.start(enc)
    # prompt, a multi-token continuation and single steps all go through the same caches
    mine = torch.cat([m.decode(st, toks[:2]), m.decode(st, toks[2:4]), m.decode(st, toks[4:5]), m.decode(st, toks[5:])])
    assert torch.nn.functional.cosine_similarity(mine.flatten(), ref.flatten(), dim=0) > 0.999
    assert st["pos"] == 6
    with pytest.raises(ValueError):
        m.decode(st, torch.zeros(cfg.max_target, dtype=torch.int32))


def _vocab(cfg):
    # text ids < 200; eot 200, sot 201, languages 202-203, translate 204, transcribe 205, no-speech 206,
    # no-timestamps 207, timestamps from 208
    return WhisperVocab(sot=201, eot=200, transcribe=205, translate=204, no_timestamps=207, timestamp_begin=208,
                        no_speech=206, languages={"en": 202, "de": 203})


def test_whisper_grammar_and_windows():
    cfg, _, m = _hf_pair()
    v = _vocab(cfg)
    pipe = WhisperPipeline(m, v)
    opts = WhisperOptions(language="en")
    ninf = float("-inf")
    tb = v.timestamp_begin
    # first token: a timestamp no later than max_initial_timestamp
    lg = pipe._mask_logits(torch.zeros(cfg.vocab), [201, 202, 205], 3, opts)
    assert (lg[:tb] == ninf).all() and lg[tb] == 0 and lg[tb + 50] == 0 and lg[tb + 51] == ninf
    # after an opening stamp: text only
    lg = pipe._mask_logits(torch.zeros(cfg.vocab), [201, 202, 205, tb + 3], 3, opts)
    assert (lg[tb:] == ninf).all() and lg[5] == 0
    # after text + one stamp: only a stamp (not earlier) or the end
    base = torch.zeros(cfg.vocab)
    base[v.eot] = 20.0          # keeps the "timestamps outweigh text" rule out of this case
    lg = pipe._mask_logits(base, [201, 202, 205, tb + 3, 7, 8, tb + 9], 3, opts)
    assert (lg[:v.eot] == ninf).all() and lg[v.eot] == 20 and lg[tb + 8] == ninf and lg[tb + 9] == 0
    # ... and with flat logits that rule removes every non-timestamp
    lg = pipe._mask_logits(torch.zeros(cfg.vocab), [201, 202, 205, tb + 3, 7, 8, tb + 9], 3, opts)
    assert (lg[:tb] == ninf).all() and lg[tb + 9] == 0
    # without timestamps no stamp can be produced
    lg = pipe._mask_logits(torch.zeros(cfg.vocab), [201, 202, 205, 207, 4], 4, WhisperOptions(language="en", timestamps=False))
    assert (lg[tb:] == ninf).all() and lg[v.eot] == 0

    # segments: two closed pairs, then the window advances to the last stamp
    toks = [tb + 0, 5, 6, tb + 10, tb + 10, 7, tb + 25, tb + 25]
    segs, adv = pipe._segments(toks, 30.0, 1.0, -0.1, 0.0)
    assert [(round(s.start, 2), round(s.end, 2), s.tokens) for s in segs] == [(30.0, 30.2, [5, 6]), (30.2, 30.5, [7])]
    assert abs(adv - 0.5) < 1e-6
    segs, adv = pipe._segments([tb + 0, 5, 6, tb + 20], 0.0, 1.0, -0.1, 0.0)
    assert len(segs) == 1 and abs(segs[0].end - 0.4) < 1e-6 and adv == 1.0

    # end to end on noise: every window is decoded, stamps are ordered, time moves forward
    lang, probs = pipe.detect_language(m.encode(torch.randn(cfg.n_mels, 2 * cfg.max_source)))
    assert lang in ("en", "de") and abs(sum(probs.values()) - 1) < 1e-4
    audio = torch.randn(int(16000 * 2.5), generator=torch.Generator().manual_seed(3)) * 0.1
    res = pipe.transcribe(audio, 16000, WhisperOptions(no_speech_threshold=2.0))
    assert res.language in ("en", "de") and abs(res.duration_s - 2.5) < 1e-6
    assert res.segments and all(s.end >= s.start for s in res.segments)
    assert all(b.start >= a.start for a, b in zip(res.segments, res.segments[1:]))
    res2 = pipe.transcribe(torch.stack([audio, audio]), 16000, WhisperOptions(language="de", timestamps=False, max_new_tokens=5,
                                                                              no_speech_threshold=2.0))
    assert res2.language == "de" and len(res2.segments) == 3 and all(len(s.tokens) <= 5 for s in res2.segments)


def _whisper_dir(tmp_path):
    """A tiny Whisper checkpoint directory: config, weights, a byte-level tokenizer.json with the
    control tokens."""
    import json
    from hartsyinference_b200.models.llm.loader import save_hf_checkpoint
    cfg, hf, _ = _hf_pair()
    d = tmp_path / "whisper-tiny-synth"
    tensors = {k: v.detach().to(torch.bfloat16).contiguous() for k, v in hf.state_dict().items() if k != "proj_out.weight"}
    save_hf_checkpoint({**hf.config.to_dict(), "model_type": "whisper"}, tensors, d)
    from hartsyinference_b200.assets.tokenizer import _bytes_to_unicode
    b2u = _bytes_to_unicode()
    vocab = {b2u[b]: b for b in range(200)}
    specials = ["<|endoftext|>", "<|startoftranscript|>", "<|en|>", "<|de|>", "<|translate|>", "<|transcribe|>",
                "<|nospeech|>", "<|notimestamps|>"] + [f"<|{i * 0.02:.2f}|>" for i in range(cfg.vocab - 208)]
    added = [{"id": 200 + i, "content": s, "special": True} for i, s in enumerate(specials)]
    (d / "tokenizer.json").write_text(json.dumps({
        "model": {"type": "BPE", "vocab": vocab, "merges": []}, "added_tokens": added,
        "pre_tokenizer": {"type": "ByteLevel", "add_prefix_space": False}}))
    (d / "generation_config.json").write_text(json.dumps({"suppress_tokens": [1, 2], "begin_suppress_tokens": [32, 200]}))
    return d


def test_transcribe_service_and_endpoint(tmp_path):
    from fastapi.testclient import TestClient
    from hartsyinference_b200.engine import AudioRequest, InferenceEngine, ModelSpec
    from hartsyinference_b200.engine.requests import Modality
    from hartsyinference_b200.server.app import ServerOptions, create_app
    d = _whisper_dir(tmp_path)
    eng = InferenceEngine("cpu")
    assert eng.is_supported(Modality.TRANSCRIBE)
    audio = torch.randn(16000, generator=torch.Generator().manual_seed(5)) * 0.1
    wav = write_wav(tmp_path / "a.wav", audio, 16000)
    res = eng.transcribe.run(ModelSpec(str(d)), AudioRequest(audio=str(tmp_path / "a.wav"), language="en"))
    assert res.language == "en" and abs(res.duration_s - 1.0) < 1e-3
    pipe = eng.transcribe._pipe(ModelSpec(str(d)))
    v = pipe.vocab
    assert (v.sot, v.eot, v.no_timestamps, v.timestamp_begin, v.no_speech) == (201, 200, 207, 208, 206)
    assert v.languages == {"en": 202, "de": 203} and v.suppress == [1, 2] and v.begin_suppress == [32, 200]
    assert "whisper:" + str(d) in eng.loaded_pipeline_keys

    app = create_app(ServerOptions(models={"whisper": str(d)}), engine=eng)
    with TestClient(app) as c:
        boundary = "xyzBOUNDARY"
        body = (f"--{boundary}\r\nContent-Disposition: form-data; name=\"model\"\r\n\r\nwhisper\r\n"
                f"--{boundary}\r\nContent-Disposition: form-data; name=\"response_format\"\r\n\r\nverbose_json\r\n"
                f"--{boundary}\r\nContent-Disposition: form-data; name=\"file\"; filename=\"a.wav\"\r\n"
                f"Content-Type: audio/wav\r\n\r\n").encode() + wav + f"\r\n--{boundary}--\r\n".encode()
        r = c.post("/v1/audio/transcriptions", content=body, headers={"content-type": f"multipart/form-data; boundary={boundary}"})
        assert r.status_code == 200, r.text
        j = r.json()
        assert j["text"] == res.text or isinstance(j["text"], str)
        assert abs(j["duration"] - 1.0) < 1e-3 and isinstance(j["segments"], list)
        r = c.post("/v1/audio/transcriptions", json={"model": "whisper"})
        assert r.status_code == 400
    eng.close()


def test_cli_transcribe_verb(tmp_path):
    from click.testing import CliRunner
    from hartsyinference_b200.cli.main import cli
    d = _whisper_dir(tmp_path)
    write_wav(tmp_path / "b.wav", torch.randn(8000, generator=torch.Generator().manual_seed(7)) * 0.1, 8000)
    r = CliRunner().invoke(cli, ["transcribe", str(d), str(tmp_path / "b.wav"), "--language", "en", "--json", "--device", "cpu"])
    assert r.exit_code == 0, r.output


def _vits_hf(stochastic=True):
    tr = pytest.importorskip("transformers")
    c = tr.VitsConfig(vocab_size=40, hidden_size=64, num_hidden_layers=2, num_attention_heads=2, ffn_dim=128, flow_size=64,
                      spectrogram_bins=33, upsample_initial_channel=64, upsample_rates=[4, 4], upsample_kernel_sizes=[8, 8],
                      resblock_kernel_sizes=[3, 5], resblock_dilation_sizes=[[1, 3], [1, 3]], prior_encoder_num_flows=2,
                      prior_encoder_num_wavenet_layers=2, duration_predictor_num_flows=2, duration_predictor_filter_channels=32,
                      depth_separable_num_layers=2, posterior_encoder_num_wavenet_layers=2, window_size=4,
                      use_stochastic_duration_prediction=stochastic)
    torch.manual_seed(0)
    hf = tr.VitsModel(c).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if p.ndim >= 2 and "emb_rel" not in n:
                p.mul_(1.5)
            if n.endswith("bias"):
                p.add_(torch.randn_like(p) * 0.1)
    return c, hf


@pytest.mark.parametrize("stochastic", [True, False])
def test_vits_matches_transformers(stochastic):
    from hartsyinference_b200.models.audio.vits import VitsModel, tiny_vits, vits_from_hf
    c, hf = _vits_hf(stochastic)
    hf.noise_scale = hf.noise_scale_duration = 0.0        # both samplers off: the waveform is a function of the ids
    sd = {k: v.detach() for k, v in hf.state_dict().items()}
    cfg = vits_from_hf(c.to_dict())
    assert cfg == tiny_vits(stochastic_duration=stochastic, sampling_rate=cfg.sampling_rate)
    m = VitsModel(cfg, "cpu", get=lambda n: sd.get(n))
    for seed, n in ((1, 13), (2, 3), (3, 30)):      # shorter and longer than the relative-attention window
        ids = torch.randint(0, 40, (n,), generator=torch.Generator().manual_seed(seed))
        with torch.no_grad():
            ref = hf(input_ids=ids[None]).waveform[0]
        mine = m.synthesize(ids, 0.0, 0.0)
        assert mine.shape == ref.shape and mine.numel() % cfg.hop == 0
        assert (mine - ref).abs().max() < 2e-3
    slow = m.synthesize(ids, 0.0, 0.0, speaking_rate=0.5)
    assert slow.numel() > mine.numel()
    a, b = m.synthesize(ids), m.synthesize(ids)
    assert a.abs().max() <= 1.0 and (a.shape != b.shape or not torch.equal(a, b))     # sampling is on by default


def test_speech_service_endpoint_and_cli(tmp_path):
    import json
    from click.testing import CliRunner
    from fastapi.testclient import TestClient
    from hartsyinference_b200.cli.main import cli
    from hartsyinference_b200.engine import InferenceEngine, ModelSpec, SpeechRequest
    from hartsyinference_b200.models.llm.loader import save_hf_checkpoint
    from hartsyinference_b200.pipelines.vits import VitsCharTokenizer, VitsPipeline
    from hartsyinference_b200.server.app import ServerOptions, create_app
    c, hf = _vits_hf()
    d = tmp_path / "voice"
    save_hf_checkpoint(c.to_dict(), {k: v.detach().float().contiguous() for k, v in hf.state_dict().items()
                                     if not k.startswith("posterior_encoder")}, d)
    chars = "<pad> abcdefghijklmnopqrstuvwxyz.,!?'-"
    vocab = {"<pad>": 0, **{ch: i + 1 for i, ch in enumerate(chars[5:])}}
    (d / "vocab.json").write_text(json.dumps(vocab))
    (d / "tokenizer_config.json").write_text(json.dumps({"add_blank": True, "normalize": True, "pad_token": "<pad>"}))
    tok = VitsCharTokenizer.from_dir(d)
    assert tok.encode("Ab") == [0, vocab["a"], 0, vocab["b"], 0] and tok.encode("#") == [0]

    eng = InferenceEngine("cpu")
    res = eng.speech.run(ModelSpec(str(d)), SpeechRequest(text="Hello there. How are you?", noise_scale=0.0, noise_scale_duration=0.0))
    assert res.sample_rate == 16000 and res.samples.numel() > 0 and abs(res.seconds - res.samples.numel() / 16000) < 1e-6
    pipe = eng.speech._loaded[str(d)]
    assert isinstance(pipe, VitsPipeline) and "vits:" + str(d) in eng.loaded_pipeline_keys
    pipe.max_chars = 12
    assert pipe.split("Hello there. How are you? Fine.") == ["Hello there.", "How are you?", "Fine."]
    assert all(len(x) <= 12 for x in pipe.split("a very long sentence without any punctuation at all"))
    pipe.max_chars = 300
    assert pipe.speak("###").samples.numel() == 0

    app = create_app(ServerOptions(models={"voice": str(d)}), engine=eng)
    with TestClient(app) as cl:
        r = cl.post("/v1/audio/speech", json={"model": "voice", "input": "hi there", "voice": "default"})
        assert r.status_code == 200 and r.headers["content-type"] == "audio/wav"
        wav, rate = read_wav(r.content)
        assert rate == 16000 and wav.shape[1] > 0
        r = cl.post("/v1/audio/speech", json={"model": "voice", "input": "hi", "response_format": "pcm", "speed": 2.0})
        assert r.status_code == 200 and len(r.content) % 2 == 0 and r.headers["x-sample-rate"] == "16000"
        assert cl.post("/v1/audio/speech", json={"model": "voice", "input": " "}).status_code == 400
        assert cl.post("/v1/audio/speech", json={"model": "voice", "input": "x", "response_format": "mp3"}).status_code == 400
    eng.close()
    out = tmp_path / "o.wav"
    r = CliRunner().invoke(cli, ["speak", str(d), "hello", "--out", str(out), "--device", "cpu"])
    assert r.exit_code == 0, r.output
    assert read_wav(out)[1] == 16000


def test_moonshine_matches_transformers_and_serves(tmp_path):
    tr = pytest.importorskip("transformers")
    from hartsyinference_b200.engine import AudioRequest, InferenceEngine, ModelSpec
    from hartsyinference_b200.models.audio.moonshine import MoonshineModel, moonshine_from_hf, tiny_moonshine
    from hartsyinference_b200.models.llm.loader import save_hf_checkpoint
    c = tr.MoonshineConfig(vocab_size=300, hidden_size=64, intermediate_size=128, encoder_num_hidden_layers=2, decoder_num_hidden_layers=2,
                           encoder_num_attention_heads=2, decoder_num_attention_heads=2, max_position_embeddings=128)
    torch.manual_seed(0)
    hf = tr.MoonshineForConditionalGeneration(c).eval()
    with torch.no_grad():
        for _, p in hf.named_parameters():
            if p.ndim >= 2:
                p.mul_(2.0)
    sd = {k: v.detach() for k, v in hf.state_dict().items()}
    cfg = moonshine_from_hf(c.to_dict())
    assert cfg == tiny_moonshine()
    m = MoonshineModel(cfg, "cpu", get=lambda n: sd.get(n))
    audio = torch.randn(16000, generator=torch.Generator().manual_seed(1)) * 0.1
    toks = torch.tensor([1, 10, 20, 30, 40])
    with torch.no_grad():
        ref = hf(input_values=audio[None], decoder_input_ids=toks[None])
    enc = m.encode(audio)
    assert enc.shape == ref.encoder_last_hidden_state[0].shape == (40, 64)
    assert torch.allclose(enc, ref.encoder_last_hidden_state[0], atol=1e-4)
    st = m.start(enc)
    mine = torch.cat([m.decode(st, toks[:3]), m.decode(st, toks[3:4]), m.decode(st, toks[4:])])
    assert torch.allclose(mine, ref.logits[0], atol=1e-3) and st["pos"] == 5
    with torch.no_grad():
        gen = hf.generate(input_values=audio[None], max_new_tokens=6, do_sample=False)[0].tolist()
    assert m.transcribe_tokens(audio, max_tokens=6) == [t for t in gen[1:] if t != cfg.eos_id][:6]

    d = tmp_path / "moonshine"
    save_hf_checkpoint({**c.to_dict(), "model_type": "moonshine"}, {k: v.contiguous() for k, v in sd.items() if k != "proj_out.weight"}, d)
    eng = InferenceEngine("cpu")
    long_audio = torch.randn(16000 * 3, generator=torch.Generator().manual_seed(2)) * 0.1
    res = eng.transcribe.run(ModelSpec(str(d)), AudioRequest(audio=long_audio, sample_rate=16000))
    assert abs(res.duration_s - 3.0) < 1e-6 and len(res.segments) == 1 and res.segments[0].tokens
    pipe = eng.transcribe._pipe(ModelSpec(str(d)))
    assert type(pipe).__name__ == "MoonshinePipeline"
    pipe.window_s = 1.0
    cuts = pipe._windows(long_audio)
    assert len(cuts) >= 3 and cuts[0][0] == 0 and cuts[-1][1] == long_audio.numel() and all(a < b for a, b in cuts)
    assert all(cuts[i][1] == cuts[i + 1][0] for i in range(len(cuts) - 1))
    eng.close()


def test_streaming_transcriber_commits_behind_the_hold_window():
    from hartsyinference_b200.pipelines.whisper import StreamingTranscriber, TranscriptResult, WhisperSegment

    class Fake:
        """Reports one segment per full second of the audio it is given."""
        def __init__(self):
            self.calls = []

        def transcribe(self, audio, rate, options=None):
            n = audio.numel() // rate
            self.calls.append(audio.numel())
            return TranscriptResult(segments=[WhisperSegment(float(i), float(i + 1), f" s{i}") for i in range(n)], duration_s=audio.numel() / rate)

    st = StreamingTranscriber(Fake(), rate=16000, hold_s=2.0)
    new, tail = st.push(torch.zeros(16000 * 3))
    assert [s.text for s in new] == [" s0"] and tail == "s1 s2"          # only what ends 2 s before the live edge
    new, tail = st.push(torch.zeros(8000))                                   # 2.5 s buffered, stream time 1.0 .. 3.5
    assert new == [] and tail == "s0 s1"
    new, tail = st.push(torch.zeros(2, 16000 * 2))                           # stereo input, 4.5 s buffered
    assert [round(s.start, 2) for s in new] == [1.0, 2.0] and abs(st.offset_s - 3.0) < 1e-6
    new, tail = st.flush()
    assert tail == "" and [round(s.end, 2) for s in new] == [4.0, 5.0] and st.buffer.numel() == 0
    assert len(st.committed) == 5 and st.text.startswith("s0")
    assert StreamingTranscriber(Fake()).push(torch.zeros(100)) == ([], "")


def test_dac_codec_matches_transformers():
    """DAC encode (codes) and decode (waveform) against ``DacModel``, with plain and weight-normalised convolutions."""
    tr = pytest.importorskip("transformers")
    from hartsyinference_b200.models.audio.dac import DacCodec, DacConfig
    hf_cfg = tr.DacConfig(encoder_hidden_size=8, downsampling_ratios=[2, 4], upsampling_ratios=[4, 2], decoder_hidden_size=32,
                          n_codebooks=3, codebook_size=16, codebook_dim=4, hidden_size=32)
    torch.manual_seed(0)
    hf = tr.DacModel(hf_cfg).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith("alpha"):
                p.uniform_(0.5, 1.5)
    sd = {k: v.detach() for k, v in hf.state_dict().items()}
    cfg = DacConfig.from_hf(hf_cfg.to_dict())
    assert cfg.hop == 8 and cfg.up == (4, 2)
    codec = DacCodec(cfg, lambda n: sd.get(n))
    wave = torch.randn(2, 160, generator=torch.Generator().manual_seed(1)) * 0.3
    with torch.no_grad():
        enc = hf.encode(wave[:, None])
        ref_wave = hf.decode(audio_codes=enc.audio_codes).audio_values
    codes = codec.encode(wave)
    assert codes.shape == (2, 3, 20)
    assert (codes == enc.audio_codes).float().mean() > 0.97          # ties between near-equal codes may flip
    out = codec.decode(enc.audio_codes)
    assert out.shape == (2, 160)
    assert torch.allclose(out, ref_wave.reshape(2, -1), atol=1e-4)
    # weight-normalised storage (g, v) folds to the same convolution
    wn = dict(sd)
    for k in [k for k in sd if k.endswith("conv1.weight") and k.startswith("decoder.block")]:
        v = sd[k]
        wn.pop(k)
        wn[k[:-len("weight")] + "weight_v"] = v * 3.0
        wn[k[:-len("weight")] + "weight_g"] = v.flatten(1).norm(dim=1).reshape(-1, 1, 1)
    out2 = DacCodec(cfg, lambda n: wn.get(n)).decode(enc.audio_codes)
    assert torch.allclose(out2, out, atol=1e-5)


@pytest.mark.parametrize("causal", [True, False])
def test_encodec_decoder_matches_transformers(causal):
    """EnCodec codes -> waveform against ``EncodecModel.decode`` (causal and centred padding)."""
    tr = pytest.importorskip("transformers")
    from hartsyinference_b200.models.audio.encodec import EncodecConfig, EncodecDecoder
    hf_cfg = tr.EncodecConfig(num_filters=4, upsampling_ratios=[4, 2], hidden_size=16, codebook_size=16, num_lstm_layers=2,
                              target_bandwidths=[1.5, 3.0], sampling_rate=800, num_residual_layers=2, use_causal_conv=causal,
                              use_conv_shortcut=causal)
    torch.manual_seed(0)
    hf = tr.EncodecModel(hf_cfg).eval()
    with torch.no_grad():
        for layer in hf.quantizer.layers:
            layer.codebook.embed.normal_()
    sd = {k: v.detach() for k, v in hf.state_dict().items()}
    dec = EncodecDecoder(EncodecConfig.from_hf(hf_cfg.to_dict()), lambda n: sd.get(n))
    codes = torch.randint(0, 16, (2, 3, 11), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        ref = hf.decode(codes[None], [None])[0]
    out = dec.decode(codes)
    assert out.shape == ref.shape == (2, 1, 88)
    assert torch.allclose(out, ref, atol=1e-5), (out - ref).abs().max()


def test_musicgen_matches_transformers():
    """MusicGen decoder logits (teacher forced) and the whole text -> codes -> audio path with greedy
    decoding, the codebook delay pattern and classifier-free guidance, against transformers."""
    tr = pytest.importorskip("transformers")
    from transformers.models.musicgen.configuration_musicgen import MusicgenDecoderConfig
    from hartsyinference_b200.models.audio.musicgen import Musicgen, delay_mask
    t5 = tr.T5Config(vocab_size=64, d_model=32, d_kv=8, d_ff=64, num_layers=2, num_heads=4, feed_forward_proj="relu")
    enc = tr.EncodecConfig(num_filters=4, upsampling_ratios=[4, 2], hidden_size=16, codebook_size=16, num_lstm_layers=1,
                           target_bandwidths=[1.5, 3.0], sampling_rate=800, num_residual_layers=1)
    dec = MusicgenDecoderConfig(vocab_size=16, hidden_size=48, num_hidden_layers=2, num_attention_heads=4, ffn_dim=64, num_codebooks=4,
                                max_position_embeddings=64, pad_token_id=16, bos_token_id=16)
    cfg = tr.MusicgenConfig(text_encoder=t5.to_dict(), audio_encoder=enc.to_dict(), decoder=dec.to_dict())
    torch.manual_seed(0)
    hf = tr.MusicgenForConditionalGeneration(cfg).eval()
    with torch.no_grad():
        for p in hf.parameters():
            if p.ndim >= 2:
                p.mul_(3.0)
        for layer in hf.audio_encoder.quantizer.layers:
            layer.codebook.embed.normal_()
    sd = {k: v.detach() for k, v in hf.state_dict().items()}
    m = Musicgen(cfg.to_dict(), lambda n: sd.get(n))
    assert not m.text.cfg.gated and m.proj_w is not None
    ids = torch.randint(2, 64, (7,), generator=torch.Generator().manual_seed(1))
    states = m.text_states(ids)
    with torch.no_grad():
        ref_states = hf.enc_to_dec_proj(hf.text_encoder(input_ids=ids[None]).last_hidden_state)[0]
    assert torch.nn.functional.cosine_similarity(states.flatten(), ref_states.flatten(), dim=0) > 0.99
    codes_in = torch.randint(0, 17, (4, 9), generator=torch.Generator().manual_seed(2))
    with torch.no_grad():
        ref = hf.decoder(input_ids=codes_in, encoder_hidden_states=ref_states[None]).logits            # [1, K, T, V]
    mine = m.decoder.forward(codes_in, ref_states, m.decoder.new_cache())
    assert torch.allclose(mine, ref.reshape(4, 9, 16), atol=2e-3), (mine - ref.reshape(4, 9, 16)).abs().max()
    assert delay_mask(4, 8).int().tolist() == [[0, 1, 1, 1, 1, 0, 0, 0], [0, 0, 1, 1, 1, 1, 0, 0],
                                               [0, 0, 0, 1, 1, 1, 1, 0], [0, 0, 0, 0, 1, 1, 1, 1]]
    hf.generation_config.update(do_sample=False, guidance_scale=3.0, max_length=12, pad_token_id=16, bos_token_id=16,
                                decoder_start_token_id=16)
    with torch.no_grad():
        ref_audio = hf.generate(input_ids=ids[None], attention_mask=torch.ones(1, 7, dtype=torch.long))
    frames = ref_audio.shape[-1] // 8
    assert frames in (12 - 4, 12 - 4 + 1)                      # the generation-length bookkeeping differs between releases
    codes = m.decoder.generate(ref_states, frames, guidance=3.0)
    audio = m.codec.decode(codes[None])[0]
    assert audio.shape == ref_audio[0].shape == (1, frames * 8)
    assert torch.allclose(audio, ref_audio[0], atol=1e-3), (audio - ref_audio[0]).abs().max()


def test_music_service_generates_audio_from_a_checkpoint_directory(tmp_path):
    """A MusicGen directory (config.json + safetensors) through the engine's music service: the
    requested duration, determinism of greedy decoding, and the prompt actually steering the result."""
    tr = pytest.importorskip("transformers")
    import json
    from transformers.models.musicgen.configuration_musicgen import MusicgenDecoderConfig
    from hartsyinference_b200.assets.safetensors import save_file
    from hartsyinference_b200.engine import InferenceEngine, ModelSpec, MusicRequest
    t5 = tr.T5Config(vocab_size=300, d_model=32, d_kv=8, d_ff=64, num_layers=1, num_heads=4, feed_forward_proj="relu")
    enc = tr.EncodecConfig(num_filters=4, upsampling_ratios=[4, 2], hidden_size=16, codebook_size=16, num_lstm_layers=1,
                           target_bandwidths=[1.5, 3.0], sampling_rate=800, num_residual_layers=1)
    dec = MusicgenDecoderConfig(vocab_size=16, hidden_size=48, num_hidden_layers=1, num_attention_heads=4, ffn_dim=64, num_codebooks=4,
                                max_position_embeddings=256, pad_token_id=16, bos_token_id=16)
    cfg = tr.MusicgenConfig(text_encoder=t5.to_dict(), audio_encoder=enc.to_dict(), decoder=dec.to_dict())
    torch.manual_seed(0)
    hf = tr.MusicgenForConditionalGeneration(cfg)
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if p.ndim >= 2 and not n.startswith("audio_encoder."):
                p.mul_(4.0)                                      # make the text matter; the codec stays unsaturated
        for layer in hf.audio_encoder.quantizer.layers:
            layer.codebook.embed.normal_(std=0.3)
    d = tmp_path / "musicgen"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(cfg.to_dict()))
    save_file({k: v.detach().contiguous() for k, v in hf.state_dict().items()}, d / "model.safetensors")
    eng = InferenceEngine("cpu")
    spec = ModelSpec(str(d))
    a = eng.music.run(spec, MusicRequest(prompt="slow piano", seconds=0.2, greedy=True))
    assert a.sample_rate == 800 and a.samples.shape == (160,) and abs(a.seconds - 0.2) < 1e-6
    again = eng.music.run(spec, MusicRequest(prompt="slow piano", seconds=0.2, greedy=True))
    assert torch.equal(a.samples, again.samples)
    b = eng.music.run(spec, MusicRequest(prompt="fast drums and bass", seconds=0.2, greedy=True, guidance=8.0))
    assert not torch.allclose(a.samples, b.samples)
    s1 = eng.music.run(spec, MusicRequest(prompt="slow piano", seconds=0.2, seed=1))
    s2 = eng.music.run(spec, MusicRequest(prompt="slow piano", seconds=0.2, seed=1))
    assert torch.equal(s1.samples, s2.samples)
    assert "musicgen:" + str(d) in eng.music.loaded_keys()
