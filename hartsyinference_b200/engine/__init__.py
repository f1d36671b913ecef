"""Engine layer: continuous-batching LLM engine, diffusion services, placement planner, gates."""
from .llm_engine import LLMEngine, Request  # noqa: F401
from .sampling import SamplingParams  # noqa: F401
from .requests import (  # noqa: F401
    AudioRequest, MusicRequest, EngineOptions, RestoreRequest, ImageRequest, ModelSpec, SpeechRequest, TextRequest, TextResult, VideoRequest, VisionRequest,
)


def __getattr__(name):
    # the facade pulls in the diffusion stack; import it on first use
    if name == "InferenceEngine":
        from .inference_engine import InferenceEngine
        return InferenceEngine
    raise AttributeError(name)
