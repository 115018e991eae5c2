"""Error types of the engine.

The reference keeps one error enum with variants such as ``WeightNotFound``,
``UnsupportedModel``, ``InvalidShape`` and ``ShapeMismatch``
(infernum/src/error.rs:10-67).  Here each family of failure is an exception
class, so callers can catch exactly what they can handle.
"""

from __future__ import annotations


class InfernumError(Exception):
    """Base class of every error this package raises on purpose."""


class ConfigError(InfernumError):
    """config.json is missing a key, has a wrong type or an unsupported value."""


class UnsupportedModelError(ConfigError):
    """``model_type`` names an architecture that is not registered."""


class WeightError(InfernumError):
    """Tensors in a checkpoint do not match what the model declares.

    ``missing``, ``unexpected`` and ``wrong_shape`` hold the full lists so a
    caller can report all faults of a checkpoint at once.
    """

    def __init__(self, message, missing=(), unexpected=(), wrong_shape=(), wrong_dtype=()):
        super().__init__(message)
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)


class CacheError(InfernumError):
    """Misuse of the cache manager: double free, unknown page, unknown request."""


class OutOfPagesError(CacheError):
    """A request needs more pages than the pool can ever (or currently) give."""


class KernelError(InfernumError):
    """A CUDA kernel refused its arguments, or the extension is not available."""


class SchedulingError(InfernumError):
    """A request can never be run with the engine's limits."""
