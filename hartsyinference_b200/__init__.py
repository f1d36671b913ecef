"""hartsyinference_b200: a Blackwell (sm_100a) multimodal inference engine.

Layers, bottom up: ``ops`` (hand-written CUDA kernels + CPU oracle), ``parallel`` (symmetric heap,
fused compute+collective kernels, TP/SP/EP/CFG/PP plans), ``assets`` (safetensors / GGUF /
tokenizers), ``models`` (LLM, image DiT, video DiT, encoders, VAEs), ``engine`` (paged KV,
continuous-batching scheduler, services, placement planner), ``server`` / ``cli`` / the C ABI.
"""
__version__ = "0.1.0"

from . import config, exceptions, log  # noqa: F401
