"""Typed errors of the library.

The classes follow the error kinds of the reference's runtime
(crates/model-runtime/src/lib.rs:12-31: Memory, Context, Cancelled, Poisoned,
Invalid, Unsupported) and of its facade (crates/llama-rs/src/lib.rs: Options).
"""
from __future__ import annotations


class LlamaError(Exception):
    """Base class of every error this library raises on purpose."""


class InvalidError(LlamaError):
    """A value that can never be right: a bad config key, a bad token id, a bad step."""


class UnsupportedError(LlamaError):
    """A well-formed request for something this library does not implement."""


class OptionsError(LlamaError):
    """Bad sampling or generation options (llama-rs Error::Options)."""


class ContextError(LlamaError):
    """A sequence would outgrow its capacity; nothing was run and no state changed."""

    def __init__(self, capacity: int, requested: int):
        super().__init__(f"context capacity {capacity} exceeded: {requested} tokens requested")
        self.capacity = capacity
        self.requested = requested


class CacheMemoryError(LlamaError):
    """The cache has no free slot or not enough free pages for the step."""


class CancelledError(LlamaError):
    """The cancellation flag was set between two steps."""


class PoisonedError(LlamaError):
    """A device error left the session unusable until reset()."""


class KernelUnavailableError(LlamaError):
    """The CUDA extension is missing or could not be built: there is no CPU fallback."""


class WeightError(LlamaError):
    """Checkpoint tensors do not fit the model: one error that lists everything wrong."""

    def __init__(self, missing=(), unexpected=(), wrong_shape=(), other=()):
        self.missing = sorted(missing)
        self.unexpected = sorted(unexpected)
        self.wrong_shape = sorted(wrong_shape)  # (name, expected, got)
        self.other = list(other)
        lines = []
        if self.missing:
            lines.append("missing tensors: " + ", ".join(self.missing))
        if self.unexpected:
            lines.append("unexpected tensors: " + ", ".join(self.unexpected))
        for name, want, got in self.wrong_shape:
            lines.append(f"{name}: expected {list(want)}, got {list(got)}")
        lines.extend(self.other)
        super().__init__("; ".join(lines) if lines else "weight error")
