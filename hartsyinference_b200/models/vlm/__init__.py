"""Vision-language models: a vision tower whose patch features are projected into the decoder's
embedding space and spliced into the prompt."""
from .llava import LlavaModel  # noqa: F401
from .llava_next import LlavaNextModel, select_best_resolution  # noqa: F401
