"""Interfaces of the parts a decoder is put together from, and the plan that names them.

A *plan* is pure data: which parts each layer has (by registered kind name and
parameters), which checkpoint names their tensors have, and the order in which
layers run. The engine builds parts from a plan through the registry; a part
gets its sizes and constants as constructor arguments and never learns which
model it is in.

Shapes: T = tokens of the step (all sequences packed one after another),
h = hidden size. The residual stream is float32 [T, h] in both precisions;
activations between kernels have the runtime's dtype (float32 or bfloat16).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Optional, Tuple

import torch

from ..weights.loader import TensorSpec


# --------------------------------------------------------------------------- plan (data)
@dataclass(frozen=True)
class PartSpec:
    """A part by registered kind, its constructor parameters, and where its tensors live."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)
    prefix: str = ""  # checkpoint name = prefix + the part's own tensor name
    names: Mapping[str, str] = field(default_factory=dict)  # own name -> full checkpoint name


@dataclass(frozen=True)
class LayerSpec:
    """One layer's parts. `block` says how they are arranged (e.g. "pre_norm")."""

    block: str
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec


@dataclass(frozen=True)
class ScheduleEntry:
    """One executed layer: which layer's weights run, and on which cache entry.

    `cache` indexes the model's cache entries; two entries may name the same
    layer (weights used twice, each time with a cache entry of its own) and an
    entry with `writes_cache=False` reads the cache entry another layer filled.
    """

    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelPlan:
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding_name: str
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head_name: Optional[str]  # None: the head is the embedding table (tied)
    ignored_names: Tuple[str, ...] = ()
    stop_token_ids: Tuple[int, ...] = ()


# --------------------------------------------------------------------------- cache requests
@dataclass(frozen=True)
class KeyValueRequest:
    """A mixer whose memory grows with the sequence: keys and values per token.

    `window` None keeps every key; a number keeps the last `window` positions.
    Layers with equal requests share one storage group.
    """

    kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateRequest:
    """A mixer with per-sequence state of fixed size (zeroed when a slot is taken)."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


# --------------------------------------------------------------------------- part interfaces
class Part:
    """Base of every part: declares tensors, receives them bound to the device."""

    kind = "part"
    # True when forward() only enqueues device work (no host read of device data, no
    # host-side branching on it): then a decode step may be captured in a CUDA graph.
    graph_safe = False

    def tensors(self) -> Dict[str, TensorSpec]:
        """Own tensor names (relative to the part's prefix) and their shapes."""
        return {}

    def bind(self, weights: Dict[str, torch.Tensor], runtime) -> None:
        """Receive device tensors under the names of `tensors()`; fuse or reorder here."""


class Norm(Part):
    def forward(self, hidden: torch.Tensor, ctx, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """float32 residual [T,h] -> normalized activations [T,h] (or [len(rows),h])."""
        raise NotImplementedError


class PositionEncoding(Part):
    def rotary_table(self) -> Optional[Tuple[torch.Tensor, int]]:
        """(inverse frequencies float32 [R/2], R) when the scheme is a split-half
        rotation by position * frequency, which the cache-store kernel applies
        itself; None for every other scheme."""
        return None

    def head_permutation(self) -> Optional[List[int]]:
        """A reordering of a head's dimensions under which the scheme takes the form the kernels
        implement (new dimension j is old dimension permutation[j]), or None. The mixer applies
        it once to the rows of its query and key projections; scores do not change, because
        queries and keys are reordered alike."""
        return None

    def apply(self, q: torch.Tensor, k: torch.Tensor, ctx) -> Tuple[torch.Tensor, torch.Tensor]:
        """Any scheme that is not a rotary table transforms q and k here."""
        return q, k


class Mixer(Part):
    def cache_request(self):
        """KeyValueRequest, StateRequest or None."""
        return None

    def forward(self, x: torch.Tensor, ctx, cache, residual: torch.Tensor) -> torch.Tensor:
        """x: normalized activations [T,h]. Returns the new residual stream.

        `residual` is the float32 stream the mixer's output is added to; the
        part may add in place (a fused epilogue) and return the same tensor.
        `cache` is the view of this schedule entry's cache storage (or None).
        """
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx, residual: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    """Arrangement of one layer's parts; owns them and forwards tensors()/bind() to them."""

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, mixer_norm: Norm,
                 feed_forward_norm: Norm):
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.feed_forward_norm = feed_forward_norm

    def forward(self, hidden: torch.Tensor, ctx, cache) -> torch.Tensor:
        raise NotImplementedError
