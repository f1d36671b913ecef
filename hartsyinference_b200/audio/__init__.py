"""Audio IO and DSP front ends (WAV files, resampling, STFT, mel filterbanks, log-mel features)."""
from .dsp import hann_window, log_mel_spectrogram, mel_filterbank, stft_power  # noqa: F401
from .wav import read_wav, resample, write_wav  # noqa: F401
