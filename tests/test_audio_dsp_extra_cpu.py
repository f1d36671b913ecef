"""Output-level helpers, the YIN pitch tracker and Kaldi filter-bank features."""
import math

import pytest
import torch

from hartsyinference_b200.audio import dsp


def test_level_helpers():
    x = torch.sin(torch.arange(8000) * 0.05) * 0.2
    assert float(dsp.normalize_peak(x, 0.9).abs().max()) == pytest.approx(0.9, abs=1e-6)
    y = dsp.normalize_rms(x, 0.1)
    assert float(y.pow(2).mean().sqrt()) == pytest.approx(0.1, rel=1e-4)
    spiky = torch.zeros(8000)
    spiky[100] = 0.5
    z = dsp.normalize_rms(spiky, 0.1, peak_ceiling=0.95)                 # the RMS target would clip: the ceiling wins
    assert float(z.abs().max()) == pytest.approx(0.95, abs=1e-6)
    quiet = torch.full((100,), 1e-6)
    assert dsp.normalize_peak(quiet) is quiet and dsp.normalize_rms(quiet) is quiet


def test_yin_tracks_tones_and_marks_noise_unvoiced():
    rate, hop = 16000, 320
    t = torch.arange(rate) / rate
    for f in (110.0, 220.0, 440.0):
        tone = torch.sin(2 * math.pi * f * t) + 0.3 * torch.sin(2 * math.pi * 2 * f * t)
        f0 = dsp.estimate_f0(tone, rate, hop)
        assert f0.shape == (rate // hop,)
        mid = f0[2:-8]
        assert float((mid - f).abs().max()) < 0.01 * f, (f, mid)
    sweep = torch.sin(2 * math.pi * torch.cumsum(torch.linspace(150, 300, rate) / rate, 0))
    f0 = dsp.estimate_f0(sweep, rate, hop)
    assert float(f0[5]) < float(f0[20]) < float(f0[40]) and abs(float(f0[25]) - (150 + 150 * (25 * hop + 600) / rate)) < 12
    noise = torch.randn(rate, generator=torch.Generator().manual_seed(0)) * 0.1
    assert float((dsp.estimate_f0(noise, rate, hop) == 0).float().mean()) > 0.8
    assert dsp.estimate_f0(torch.zeros(100), rate, hop).numel() == 0


def test_kaldi_fbank_matches_torchaudio():
    kaldi = pytest.importorskip("torchaudio.compliance.kaldi")
    g = torch.Generator().manual_seed(0)
    t = torch.arange(16000) / 16000
    wave = (torch.sin(2 * math.pi * 300 * t) * 0.3 + torch.randn(16000, generator=g) * 0.05)
    want = kaldi.fbank(wave[None], num_mel_bins=80, dither=0.0, sample_frequency=16000.0)
    got = dsp.kaldi_fbank(wave, 16000, 80)
    assert got.shape == want.shape == ((16000 - 400) // 160 + 1, 80)
    assert torch.allclose(got, want, atol=2e-3), float((got - want).abs().max())
    want24 = kaldi.fbank(wave[None], num_mel_bins=40, dither=0.0, sample_frequency=24000.0, low_freq=50.0, high_freq=-200.0)
    assert torch.allclose(dsp.kaldi_fbank(wave, 24000, 40, low_freq=50.0, high_freq=-200.0), want24, atol=2e-3)
    assert dsp.kaldi_fbank(torch.zeros(100), 16000, 80).shape == (0, 80)


def test_fx_verb(tmp_path):
    from click.testing import CliRunner
    from hartsyinference_b200.audio import read_wav, write_wav
    from hartsyinference_b200.cli.main import cli
    rate = 16000
    t = torch.arange(rate) / rate
    tone = torch.sin(2 * math.pi * 200 * t) * 0.1
    clip = torch.cat([torch.zeros(rate // 2), tone, torch.zeros(rate // 2)])
    src, dst = tmp_path / "in.wav", tmp_path / "out.wav"
    write_wav(src, clip, rate)
    r = CliRunner().invoke(cli, ["fx", str(src), "--out", str(dst), "--op", "trim", "--op", "normalize-peak", "--op", "pitch",
                                 "--op", "resample", "--rate", "8000"])
    assert r.exit_code == 0, r.output
    assert "median 200." in r.output or "median 199." in r.output
    y, sr = read_wav(dst)
    y = y.flatten()
    assert sr == 8000 and 0.9 < y.numel() / sr < 1.2 and float(y.abs().max()) == pytest.approx(0.95, abs=0.03)
    assert CliRunner().invoke(cli, ["fx", str(src), "--op", "resample"]).exit_code != 0
