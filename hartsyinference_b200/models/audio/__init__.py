"""Audio models: Whisper-class encoder-decoder speech recognition, VITS text-to-speech, Moonshine speech recognition."""
from .whisper import WhisperConfig, WhisperModel, tiny_whisper, whisper_from_hf  # noqa: F401
from .vits import VitsConfig, VitsModel, tiny_vits, vits_from_hf  # noqa: F401
from .moonshine import MoonshineConfig, MoonshineModel, moonshine_from_hf, tiny_moonshine  # noqa: F401
