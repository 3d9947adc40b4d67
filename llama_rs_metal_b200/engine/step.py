"""The step function: run the tokens a step brings, as one batch, from the cache.

A step is a list of entries, one per sequence. Either every sequence is at its
first token (a *prefill* step: whole prompts of unequal lengths) or every
sequence goes on by exactly one token (a *decode* step). Everything is checked
before anything is launched or changed, so a rejected step leaves the cache as
it was (the reference validates before submitting for the same reason,
crates/model-runtime/src/session.rs:114-130). Sequences' lengths advance only
after the step's kernels are enqueued.
"""
from __future__ import annotations

from typing import List, Sequence

import torch

from ..cache import Cache
from ..errors import InvalidError, PoisonedError, UnsupportedError
from ..runtime import Runtime
from .batch import StepContext, StepEntry, pack_step
from .model import DecoderModel


def classify_step(entries: Sequence[StepEntry], lengths_before: Sequence[int]) -> str:
    """ "prefill" or "decode"; raises for an empty, mixed or malformed step."""
    if not entries:
        raise InvalidError("a step needs at least one entry")
    if any(len(e.tokens) == 0 for e in entries):
        raise InvalidError("every entry of a step brings at least one token")
    if all(n == 0 for n in lengths_before):
        return "prefill"
    if all(n > 0 for n in lengths_before) and all(len(e.tokens) == 1 for e in entries):
        return "decode"
    raise UnsupportedError(
        "the sequences of a step either all start at their first token or all go on by one token")


def validate_entries(entries: Sequence[StepEntry], vocab_size: int) -> None:
    seen = set()
    for e in entries:
        if e.slot in seen:
            raise InvalidError(f"slot {e.slot} appears twice in one step")
        seen.add(e.slot)
        for t in e.tokens:
            if not 0 <= int(t) < vocab_size:
                raise InvalidError("token outside vocabulary")  # session.rs:125-130
        for p in e.want:
            if not 0 <= int(p) < len(e.tokens):
                raise InvalidError(f"wanted place {p} is outside the {len(e.tokens)} tokens of the entry")


class StepRunner:
    """Binds a model and a cache and runs steps on the current CUDA stream."""

    def __init__(self, model: DecoderModel, cache: Cache, runtime: Runtime):
        self.model, self.cache, self.runtime = model, cache, runtime
        self.poisoned = False
        self.steps_run = 0

    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """float32 logits [wanted places, vocab] on the device, in entry order then `want` order."""
        if self.poisoned:
            raise PoisonedError("a device error poisoned this session; reset it")
        entries = list(entries)
        cache = self.cache
        validate_entries(entries, self.model.plan.vocab_size)
        before = [cache.length(e.slot) for e in entries]
        phase = classify_step(entries, before)
        growth = [(e.slot, n + len(e.tokens)) for e, n in zip(entries, before)]
        cache.check_growth(growth)  # raises before anything changes
        ctx = pack_step(entries, before, self.runtime, phase)
        cache.grow(growth)
        cache.sync()
        try:
            logits = self.model.forward(ctx, cache)
        except Exception:
            self.poisoned = True
            raise
        cache.commit(growth)
        self.steps_run += 1
        return logits
