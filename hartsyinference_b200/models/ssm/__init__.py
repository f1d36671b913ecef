"""State-space language models (recurrent state instead of a KV cache)."""
from .mamba import MambaConfig, MambaModel, MambaState, tiny_mamba  # noqa: F401
from .mamba2 import Mamba2Config, Mamba2Model, mamba2_from_hf, tiny_mamba2  # noqa: F401
from .rwkv import RwkvConfig, RwkvModel, rwkv_from_hf, tiny_rwkv  # noqa: F401
from .qwen35 import Qwen35Config, Qwen35Model, qwen35_from_hf  # noqa: F401
