"""HTTP server: native routes, OpenAI-compatible routes, health, metrics."""
from .app import ServerOptions, create_app  # noqa: F401
