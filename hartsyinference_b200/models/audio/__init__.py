"""Audio models: Whisper-class encoder-decoder speech recognition, VITS text-to-speech."""
from .whisper import WhisperConfig, WhisperModel, tiny_whisper, whisper_from_hf  # noqa: F401
from .vits import VitsConfig, VitsModel, tiny_vits, vits_from_hf  # noqa: F401
