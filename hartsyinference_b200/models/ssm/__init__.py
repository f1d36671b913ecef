"""State-space language models (recurrent state instead of a KV cache)."""
from .mamba import MambaConfig, MambaModel, MambaState, tiny_mamba  # noqa: F401
