"""Wake-word chain: mel front end against a direct DFT, the embedding backbone's shapes and activation, head layout
discovery, trainer -> exported head equality and learning, the streaming contract of the detector (warm-up, chunking
independence, smoothing, refractory time, reset), the voice-activity model against torch's LSTM cell, and the Wyoming
endpoint end to end on a loopback socket."""
import asyncio
import math

import pytest
import torch
import torch.nn.functional as F

from hartsyinference_b200.audio import wake as W


def _speechlike(seconds: float, seed: int, f0: float = 140.0) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    t = torch.arange(int(seconds * W.RATE)) / W.RATE
    x = sum(torch.sin(2 * math.pi * f0 * k * t + float(torch.rand(1, generator=g)) * 6.28) / k for k in range(1, 12))
    x = x * (0.5 + 0.5 * torch.sin(2 * math.pi * 3.0 * t)) + 0.05 * torch.randn(t.numel(), generator=g)
    return x / x.abs().max() * 12000.0


def test_mel_matches_a_direct_dft():
    mel = W.WakeMel()
    x = _speechlike(0.5, 0)
    out = mel(x)[0]
    frames = W.WakeMel.frame_count(x.numel())
    assert out.shape == (frames, 32) and frames == math.ceil(x.numel() / 160 - 3)
    win = torch.hann_window(512, periodic=True, dtype=torch.float64)
    power = torch.stack([torch.fft.rfft(x[i * 160:i * 160 + 512].double() * win).abs() ** 2 for i in range(frames)])
    db = 10 * torch.log10((power.float() @ mel.mel).clamp_min(1e-10))
    want = torch.maximum(db, db.max() - 80) / 10 + 2
    assert torch.allclose(out, want, atol=2e-3)
    assert W.WakeMel.frame_count(W.CHUNK + W.LEFT_CONTEXT) == 8
    with pytest.raises(ValueError):
        mel(torch.zeros(400))
    # the floor is a reduction over the buffer: a loud event elsewhere in it lifts the quiet frames
    quiet = torch.cat([x[:1760] * 1e-4, x[:1760]])
    assert float(mel(quiet)[0][:4].min()) > float(mel(x[:1760] * 1e-4)[0][:4].min())


def test_embedding_backbone_shapes_names_and_activation():
    emb = W.SpeechEmbedding(seed=1)
    e = emb(torch.randn(3, 76, 32))
    assert e.shape == (3, 96)
    with pytest.raises(ValueError):
        emb(torch.randn(1, 75, 32))
    # the same weights under the names of the published file load to the same function
    named = {}
    for i, (w, b) in enumerate(emb.convs):
        stem = "model/conv2d/Conv2D" if i == 0 else f"model/conv2d_{i}/Conv2D"
        named[stem + "_weights_fused_bn"], named[stem + "_bias_fused_bn"] = w, b
    named["model/conv2d_19/Conv2D/ReadVariableOp:0"] = emb.final
    again = W.SpeechEmbedding(named)
    x = torch.randn(2, 76, 32)
    assert torch.equal(again(x), emb(x))
    # clipped leaky ReLU: the first layer's output never falls below -0.4
    w, b = emb.convs[0]
    y = F.leaky_relu(F.conv2d(x[:, None] * 50, w, b, padding=(0, 1)), 0.2).clamp_min(-0.4)
    assert float(y.min()) == pytest.approx(-0.4)
    clip = W.WakeMel()(_speechlike(2.0, 3))[0]
    assert emb.windows(clip).shape == ((clip.shape[0] - 76) // 8 + 1, 96)


def test_head_layout_is_read_off_the_names():
    g = torch.Generator().manual_seed(0)
    r = lambda *s: torch.randn(*s, generator=g) * 0.05
    plain = {"1.weight": r(32, 1536), "1.bias": r(32), "3.weight": r(32, 32), "3.bias": r(32), "5.weight": r(1, 32), "5.bias": r(1)}
    normed = {"model.1.weight": r(32, 1536), "model.1.bias": r(32), "model.2.weight": torch.ones(32) + r(32), "model.2.bias": r(32),
              "model.4.weight": r(32, 32), "model.4.bias": r(32), "model.5.weight": torch.ones(32), "model.5.bias": r(32),
              "model.7.weight": r(1, 32), "model.7.bias": r(1), "verifier_model.0.weight": r(4, 4)}
    x = torch.randn(5, 16, 96, generator=g)
    f = x.reshape(5, -1)
    a = W.WakeHead("alexa", plain)
    want = torch.sigmoid(F.linear(F.relu(F.linear(F.relu(F.linear(f, plain["1.weight"], plain["1.bias"])), plain["3.weight"], plain["3.bias"])),
                                  plain["5.weight"], plain["5.bias"]))[:, 0]
    assert torch.allclose(a(x), want, atol=1e-6)
    b = W.WakeHead("jarvis", normed)
    h = F.relu(F.layer_norm(F.linear(f, normed["model.1.weight"], normed["model.1.bias"]), (32,), normed["model.2.weight"], normed["model.2.bias"]))
    h = F.relu(F.layer_norm(F.linear(h, normed["model.4.weight"], normed["model.4.bias"]), (32,), normed["model.5.weight"], normed["model.5.bias"]))
    want = torch.sigmoid(F.linear(h, normed["model.7.weight"], normed["model.7.bias"]))[:, 0]
    assert torch.allclose(b(x), want, atol=1e-6) and [k for k, *_ in b.layers] == ["linear", "norm", "linear", "norm", "linear"]
    with pytest.raises(ValueError):
        W.WakeHead("bad", {"0.weight": r(1, 10), "0.bias": r(1)})


def test_trainer_learns_and_its_export_scores_the_same():
    mel, emb = W.WakeMel(), W.SpeechEmbedding(seed=2)
    pos = W.features_for_clips([_speechlike(2.5, s, 140.0) for s in range(3)], mel, emb)
    neg = W.features_for_clips([_speechlike(2.5, 10 + s, 310.0) for s in range(3)], mel, emb)
    assert pos.shape[1:] == (16, 96) and pos.shape[0] == neg.shape[0] > 5
    x = torch.cat([pos, neg])
    y = torch.cat([torch.ones(len(pos)), torch.zeros(len(neg))])
    tr = W.WakeHeadTrainer(hidden=32, lr=3e-3, seed=0)
    history = tr.fit(x, y, epochs=60, batch_size=16)
    assert history[-1] < 0.5 * history[0]
    p = tr.probability(x)
    assert float(p[:len(pos)].mean()) > 0.8 and float(p[len(pos):].mean()) < 0.2
    exported = tr.export()
    assert sorted(exported) == ["0.bias", "0.weight", "2.bias", "2.weight", "4.bias", "4.weight"]
    assert torch.allclose(W.WakeHead("word", exported)(x), p, atol=1e-6)


class _ConstantHead:
    """Scores from a script, to test the detector's own logic."""

    def __init__(self, name, scores):
        self.name, self.scores, self.calls = name, list(scores), 0

    def __call__(self, features):
        s = self.scores[min(self.calls, len(self.scores) - 1)]
        self.calls += 1
        return torch.tensor([s])


def test_detector_streaming_contract():
    mel, emb = W.WakeMel(), W.SpeechEmbedding(seed=4)
    audio = _speechlike(4.0, 7)
    det = W.WakeDetector(mel, emb)
    head = _ConstantHead("never", [0.0])
    det.add_word(head)
    sink = []
    assert det.push(audio, sink) == []
    # first chunk has no left context; 76 frames need 10 chunks of 8; then 16 embeddings
    chunks = audio.numel() // W.CHUNK
    assert len(sink) == chunks - 1 - 9 - 15 == head.calls
    # how the samples are cut up does not matter
    det2 = W.WakeDetector(mel, emb)
    det2.add_word(_ConstantHead("never", [0.0]))
    sink2 = []
    for i in range(0, audio.numel(), 777):
        det2.push(audio[i:i + 777], sink2)
    assert len(sink2) == len(sink) and all(torch.equal(a, b) for a, b in zip(sink, sink2))
    # each scored window is the last 16 embeddings of the windows embedded so far
    assert torch.equal(sink[1][:-1], sink[0][1:])

    # smoothing: one high step among low ones does not fire; three in a row do; then the word stays quiet
    det3 = W.WakeDetector(mel, emb)
    scripted = _ConstantHead("hey", [0.1, 0.9, 0.1, 0.1, 0.9, 0.9, 0.9, 0.9, 0.9, 0.9])
    det3.add_word(scripted, W.WakeWordSettings(threshold=0.7, smoothing=3, refractory=0.5))
    fired = det3.push(audio)
    first = (1 + 9 + 15 + 7) * W.CHUNK            # the 7th scored step completes the first run of three
    assert fired and fired[0].word == "hey" and fired[0].sample_index == first and fired[0].score == pytest.approx(0.9)
    gaps = [b.sample_index - a.sample_index for a, b in zip(fired, fired[1:])]
    assert all(g >= 0.5 * W.RATE for g in gaps)
    det3.reset()
    assert det3.consumed == 0 and det3.push(audio[:W.CHUNK * 5]) == []
    assert det3.remove_word("hey") and det3.words == []


def test_voice_activity_model_matches_torch_layers():
    vad = W.SileroVad(seed=3)
    g = torch.Generator().manual_seed(1)
    chunks = torch.randn(3, 512, generator=g) * 0.1
    cell = torch.nn.LSTMCell(128, 128)
    with torch.no_grad():
        cell.weight_ih.copy_(vad.w["lstm_cell.weight_ih"]); cell.weight_hh.copy_(vad.w["lstm_cell.weight_hh"])
        cell.bias_ih.copy_(vad.w["lstm_cell.bias_ih"]); cell.bias_hh.copy_(vad.w["lstm_cell.bias_hh"])
    h = c = torch.zeros(1, 128)
    context = torch.zeros(64)
    for ch in chunks:
        got = vad(ch)
        x = torch.cat([context, ch])
        x = torch.cat([x, x[-66:-1].flip(0)[:64]])                      # reflect 64 samples on the right
        context = ch[-64:]
        frames = torch.stack([torch.fft.rfft(x[i * 128:i * 128 + 256].double() * torch.hann_window(256, dtype=torch.float64)).abs().float()
                              for i in range(4)], 1)[None]
        y = frames
        for name, stride in (("conv1", 1), ("conv2", 2), ("conv3", 2), ("conv4", 1)):
            y = F.relu(F.conv1d(y, vad.w[name + ".weight"], vad.w[name + ".bias"], stride=stride, padding=1))
        assert y.shape == (1, 128, 1)
        with torch.no_grad():
            h, c = cell(y[:, :, 0], (h, c))
        want = torch.sigmoid(F.linear(F.relu(h), vad.w["final_conv.weight"][:, :, 0], vad.w["final_conv.bias"]))[0, 0]
        assert float(got[0]) == pytest.approx(float(want), abs=1e-4)
    vad.reset()
    assert float(vad.h.abs().sum()) == 0 and float(vad.context.abs().sum()) == 0
    with pytest.raises(ValueError):
        vad(torch.zeros(100))


def test_vad_stream_segments():
    class Scripted:
        def __init__(self, p): self.p, self.i = p, 0
        def reset(self): self.i = 0
        def __call__(self, chunk):
            v = self.p[min(self.i, len(self.p) - 1)]; self.i += 1
            return torch.tensor([v])
    probs = [0.1] * 3 + [0.9] * 10 + [0.1] * 3 + [0.8] * 4 + [0.05] * 15
    s = W.VadStream(Scripted(probs), threshold=0.5, min_silence=0.3)
    events = []
    for i in range(len(probs)):
        events += s.push(torch.zeros(512))
    assert events == [("start", 3 * 512), ("end", 20 * 512)]       # the short dip does not end the segment


def test_wyoming_endpoint_round_trip(tmp_path):
    from hartsyinference_b200.assets.safetensors import save_file
    from hartsyinference_b200.server import wyoming as Y
    mel, emb = W.WakeMel(), W.SpeechEmbedding(seed=5)
    half = mel.basis.shape[0] // 2
    save_file({"0.stft.conv_real.weight": mel.basis[:half].contiguous(), "0.stft.conv_imag.weight": mel.basis[half:].contiguous(),
               "1.melW": mel.mel.contiguous()}, tmp_path / "melspectrogram.safetensors")
    named = {}
    for i, (w, b) in enumerate(emb.convs):
        stem = "model/conv2d/Conv2D" if i == 0 else f"model/conv2d_{i}/Conv2D"
        named[stem + "_weights_fused_bn"], named[stem + "_bias_fused_bn"] = w.contiguous(), b.contiguous()
    named["model/conv2d_19/Conv2D/ReadVariableOp:0"] = emb.final.contiguous()
    save_file(named, tmp_path / "embedding_model.safetensors")
    pos = W.features_for_clips([_speechlike(3.0, s, 140.0) for s in range(2)], mel, emb)
    neg = W.features_for_clips([_speechlike(3.0, 10 + s, 310.0) for s in range(2)], mel, emb)
    tr = W.WakeHeadTrainer(hidden=32, lr=3e-3)
    tr.fit(torch.cat([pos, neg]), torch.cat([torch.ones(len(pos)), torch.zeros(len(neg))]), epochs=60, batch_size=16)
    models = W.WakeModelSet(tmp_path)
    assert models.heads == {} and models.vad() is None
    models.save_head("hey_b200", tr.export())
    assert list(W.WakeModelSet(tmp_path).heads) == ["hey_b200"]

    async def scenario():
        server = Y.WyomingWakeServer(models, "127.0.0.1", 0)
        port = await server.start()
        try:
            reader, writer = await asyncio.open_connection("127.0.0.1", port)
            writer.write(Y.encode_event("describe"))
            await writer.drain()
            kind, data, _ = await asyncio.wait_for(Y.read_event(reader), 10)
            writer.close()
            hit = await Y.stream_wav("127.0.0.1", port, _speechlike(3.0, 0, 140.0) / 32768.0, W.RATE)
            miss = await Y.stream_wav("127.0.0.1", port, _speechlike(3.0, 11, 310.0) / 32768.0, W.RATE)
            other = await Y.stream_wav("127.0.0.1", port, _speechlike(3.0, 0, 140.0) / 32768.0, W.RATE, names=["someone_else"])
            return kind, data, hit, miss, other
        finally:
            await server.stop()

    kind, data, hit, miss, other = asyncio.run(scenario())
    assert kind == "info" and [m["name"] for m in data["wake"][0]["models"]] == ["hey_b200"]
    assert hit and hit[0]["name"] == "hey_b200" and 1000 < hit[0]["timestamp"] <= 3000
    assert miss == [] and other == []


def test_wyoming_frames_and_pcm_conversion():
    from hartsyinference_b200.server import wyoming as Y

    async def parse(raw):
        r = asyncio.StreamReader()
        r.feed_data(raw)
        r.feed_eof()
        return await Y.read_event(r)

    raw = Y.encode_event("audio-chunk", {"rate": 16000, "width": 2, "channels": 1}, b"\x01\x00\x02\x00")
    assert asyncio.run(parse(raw)) == ("audio-chunk", {"rate": 16000, "width": 2, "channels": 1}, b"\x01\x00\x02\x00")
    assert asyncio.run(parse(b'{"type":"detect","data":{"names":["a"]}}\n')) == ("detect", {"names": ["a"]}, b"")
    assert asyncio.run(parse(b"")) is None
    with pytest.raises(ValueError):
        asyncio.run(parse(b"not json\n"))
    with pytest.raises(ValueError):
        asyncio.run(parse(b'{"type":"x","payload_length":999999999}\n'))
    stereo = torch.tensor([100, 300, -200, -400], dtype=torch.int16).numpy().tobytes()
    assert Y.pcm_to_mono16k(stereo, 16000, 2, 2).tolist() == [200.0, -300.0]
    assert Y.pcm_to_mono16k(bytes([128, 255]), 16000, 1, 1).tolist() == [0.0, 127 * 256.0]
    up = Y.pcm_to_mono16k(torch.zeros(800, dtype=torch.int16).numpy().tobytes(), 8000, 2, 1)
    assert abs(up.numel() - 1600) <= 2


def test_train_wake_word_stores_a_head_that_fires_on_the_phrase(tmp_path):
    from hartsyinference_b200.assets.safetensors import save_file
    mel, emb = W.WakeMel(), W.SpeechEmbedding(seed=6)
    half = mel.basis.shape[0] // 2
    save_file({"0.stft.conv_real.weight": mel.basis[:half].contiguous(), "0.stft.conv_imag.weight": mel.basis[half:].contiguous(),
               "1.melW": mel.mel.contiguous()}, tmp_path / "melspectrogram.safetensors")
    named = {"model/conv2d_19/Conv2D/ReadVariableOp:0": emb.final.contiguous()}
    for i, (w, b) in enumerate(emb.convs):
        stem = "model/conv2d/Conv2D" if i == 0 else f"model/conv2d_{i}/Conv2D"
        named[stem + "_weights_fused_bn"], named[stem + "_bias_fused_bn"] = w.contiguous(), b.contiguous()
    save_file(named, tmp_path / "embedding_model.safetensors")
    models = W.WakeModelSet(tmp_path)
    phrase = [_speechlike(0.9, s, 140.0) for s in range(2)]
    other = [_speechlike(6.0, 20 + s, 310.0) for s in range(2)]
    hiss = lambda n, seed: torch.randn(n, generator=torch.Generator().manual_seed(seed)) * 32768.0 * 10 ** (-35 / 20)
    other += [torch.cat([o[:2 * W.RATE], hiss(3 * W.RATE, 40 + i), o[2 * W.RATE:]]) for i, o in enumerate(other)]   # speech, pause, speech
    report = W.train_wake_word(models, "hey_there", phrase, other, epochs=150, hidden=64, copies=4)
    assert report["recall"] > 0.8 and report["false_accepts"] < 0.1 and (tmp_path / "hey_there.safetensors").exists()
    det = W.WakeModelSet(tmp_path).detector()
    stream = torch.cat([other[0][:3 * W.RATE], torch.zeros(int(2.2 * W.RATE)), phrase[0], torch.zeros(int(0.3 * W.RATE))])
    stream = stream + torch.randn(stream.numel(), generator=torch.Generator().manual_seed(0)) * 32768.0 * 10 ** (-35 / 20)
    fired = det.push(stream)
    assert fired and all(f.sample_index > 5 * W.RATE for f in fired)
    with pytest.raises(ValueError):
        W.train_wake_word(models, "x", [torch.zeros(100)], [], epochs=1)


def test_cli_lists_the_wake_verbs():
    from click.testing import CliRunner
    from hartsyinference_b200.cli.main import cli
    out = CliRunner().invoke(cli, ["--help"]).output
    assert all(v in out for v in ("wake-listen", "wake-client", "wake-train"))
    assert "Wyoming" in CliRunner().invoke(cli, ["wake-listen", "--help"]).output
