"""Decoder LLMs: config, transformer, loaders, MoE and MLA blocks."""
from .config import PRESETS, TransformerConfig  # noqa: F401
from .transformer import DecoderModel, ForwardBatch  # noqa: F401
