"""Typed errors raised by the library before any kernel launch.

The reference signals the same conditions with .NET exceptions
(src/DotLLM.Models/Architectures/TransformerModel.cs:137-143, 737-739;
src/DotLLM.Engine/KvCache/SimpleKvCache.cs:78-80).
"""


class DotLlmError(Exception):
    """Base class of every error this library raises on purpose."""


class ConfigError(DotLlmError):
    """config.json is missing, malformed, or describes a model this library does not build."""


class WeightsError(DotLlmError):
    """The safetensors file does not match the model: lists missing, unexpected and misshapen tensors."""


class CacheError(DotLlmError):
    """A cache slot or page was asked for, freed or addressed wrongly."""


class CacheFullError(CacheError):
    """The cache has no free slot or page for the request."""


class StepError(DotLlmError):
    """A step's input is invalid (token id, position, duplicate sequence)."""


class KernelError(DotLlmError):
    """A kernel refused its arguments, failed to launch, or the native library is unavailable."""
