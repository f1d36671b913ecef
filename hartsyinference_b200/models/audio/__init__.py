"""Audio models: Whisper-class encoder-decoder speech recognition."""
from .whisper import WhisperConfig, WhisperModel, tiny_whisper, whisper_from_hf  # noqa: F401
