"""Typed errors of the engine.

Mirrors the reference's exception set (src/HartsyInference.Core/Exceptions/:
``HartsyInferenceException``, ``OutOfVramException``, ``UnsupportedModelException``) and adds the
errors that only exist in a multi-GPU, paged-KV engine.
"""
from __future__ import annotations


class HartsyInferenceError(RuntimeError):
    """Base class of every error raised by this package."""

    code = 1


class OutOfVramError(HartsyInferenceError):
    """A device allocation could not be satisfied (requested vs free bytes are attached)."""

    code = 2

    def __init__(self, message: str, requested: int = 0, free: int = 0):
        super().__init__(message)
        self.requested = requested
        self.free = free


class UnsupportedModelError(HartsyInferenceError):
    code = 3


class UnsupportedBackendError(HartsyInferenceError):
    """Raised for backend selectors this engine does not implement (for example ``vulkan``)."""

    code = 4


class KvPoolExhaustedError(HartsyInferenceError):
    """No free KV page is left for an admission or an append."""

    code = 5


class QueueFullError(HartsyInferenceError):
    """The bounded request queue is full (the HTTP layer maps this to status 429)."""

    code = 6


class NativeLibraryError(HartsyInferenceError):
    """A native library is missing or a native call returned an error code."""

    code = 7


class DeviceWaitTimeout(HartsyInferenceError):
    """A bounded device-side wait gave up; the status word says where."""

    code = 8

    def __init__(self, message: str, kernel: int = 0, site: int = 0, detail: int = 0):
        super().__init__(message)
        self.kernel = kernel
        self.site = site
        self.detail = detail


class CommError(HartsyInferenceError):
    """A collective or a peer exchange failed (peer missing, rendezvous timeout)."""

    code = 9


class RequestCancelled(HartsyInferenceError):
    code = 10
