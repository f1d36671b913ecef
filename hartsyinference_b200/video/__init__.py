"""Video output: encoding frame tensors through an ffmpeg subprocess when one is installed, with a
numbered image-sequence fallback."""
from .io import FrameSequenceWriter, encode_video, ffmpeg_path, frames_to_uint8  # noqa: F401
