"""A small B200-native inference library for the Llama 3 dense decoder.

Public surface (after crates/llama-rs/src/lib.rs): Engine, Model, Session,
GenerationOptions, Sampling, GenerationResult, and the typed errors.
"""
from .errors import (CacheMemoryError, CancelledError, ContextError, InvalidError,
                     KernelUnavailableError, LlamaError, OptionsError, PoisonedError,
                     UnsupportedError, WeightError)
from .sampling.options import GenerationOptions, Sampling

__all__ = ["Engine", "Model", "Session", "GenerationOptions", "Sampling", "GenerationResult",
           "write_random_model", "LlamaError", "InvalidError", "UnsupportedError", "OptionsError",
           "ContextError", "CacheMemoryError", "CancelledError", "PoisonedError",
           "KernelUnavailableError", "WeightError"]


def __getattr__(name):
    # the engine imports torch-heavy modules; load them on first use
    if name in ("Engine", "Model", "Session", "write_random_model"):
        from .engine import session
        return getattr(session, name)
    if name == "GenerationResult":
        from .engine.generate import GenerationResult
        return GenerationResult
    raise AttributeError(name)
