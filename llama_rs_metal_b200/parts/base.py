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


class LayerSpec:
    """One layer: the kind of block that arranges it, and its parts by role.

    Which roles a layer has is the block's business: the registered block class names them
    and the family each belongs to (`Block.roles`), the engine builds one part per role and
    hands them to the block. The usual four (a mixer and a feed-forward, each behind a norm)
    can be given by name; any other set goes in `parts`.
    """

    __slots__ = ("block", "parts")

    def __init__(self, block: str, mixer: Optional[PartSpec] = None, feed_forward: Optional[PartSpec] = None,
                 mixer_norm: Optional[PartSpec] = None, feed_forward_norm: Optional[PartSpec] = None,
                 parts: Optional[Mapping[str, PartSpec]] = None):
        named = {"mixer": mixer, "feed_forward": feed_forward, "mixer_norm": mixer_norm,
                 "feed_forward_norm": feed_forward_norm}
        merged = {role: spec for role, spec in named.items() if spec is not None}
        merged.update(parts or {})
        object.__setattr__(self, "block", block)
        object.__setattr__(self, "parts", merged)

    def __setattr__(self, name, value):
        raise AttributeError("LayerSpec is immutable; use with_parts()")

    def __getattr__(self, role):
        # layer.mixer, layer.feed_forward_norm, ... read the part of that role
        try:
            return object.__getattribute__(self, "parts")[role]
        except KeyError:
            raise AttributeError(role) from None

    def with_parts(self, **changes: PartSpec) -> "LayerSpec":
        """A copy with some roles' parts replaced or added."""
        return LayerSpec(self.block, parts={**self.parts, **changes})

    def __repr__(self):
        return f"LayerSpec({self.block!r}, {dict(self.parts)!r})"


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
    embedding_scale: Optional[float] = None  # embedded rows are multiplied by this (None: 1)
    logit_scale: Optional[float] = None      # logits are multiplied by this (None: 1)


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
    # True when forward() adds `ctx.pending` (partial sums that belong to the residual stream,
    # see StepContext.pending) to `hidden` itself before it normalizes. A block that is about to
    # pass a part's output through such a norm may let the part leave its sums there.
    folds_pending = False

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
    """Arrangement of one layer's parts. The class says which roles a layer of this kind has
    and to which family each belongs ("mixer", "feed_forward", "norm"); the engine builds
    one part per role from the layer's LayerSpec and passes them by role name. A block with
    other roles (a norm after the mixer, a second feed-forward) overrides `roles`."""

    roles: Mapping[str, str] = {"mixer": "mixer", "feed_forward": "feed_forward",
                                "mixer_norm": "norm", "feed_forward_norm": "norm"}

    def __init__(self, **parts: Part):
        missing = [role for role in self.roles if role not in parts]
        if missing:
            raise TypeError(f"{type(self).__name__} needs parts for {', '.join(missing)}")
        self.parts: Dict[str, Part] = dict(parts)
        for role, part in parts.items():
            setattr(self, role, part)

    def cache_request(self):
        """What this layer asks of the cache (one request per layer): its mixer's."""
        mixer = self.parts.get("mixer")
        return mixer.cache_request() if mixer is not None else None

    @property
    def folds_pending_on_entry(self) -> bool:
        """True when the first thing forward() does with `hidden` is to pass it through a norm
        that folds ctx.pending (the layer before may then leave partial sums there)."""
        return False

    def forward(self, hidden: torch.Tensor, ctx, cache) -> torch.Tensor:
        raise NotImplementedError
