"""Engine layer: continuous-batching LLM engine, diffusion services, placement planner, gates."""
from .llm_engine import LLMEngine, Request  # noqa: F401
from .sampling import SamplingParams  # noqa: F401
