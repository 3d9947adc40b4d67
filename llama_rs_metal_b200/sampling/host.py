"""The reference's sampler on host logits: penalty, top-k, top-p, SplitMix64.

The reference runs everything stochastic on the CPU from the logits it copied
back (crates/llama-rs/src/generation.rs:33-46; crates/llama-rs/src/sampling.rs:37-120);
this module is that sampler, in float64 like the original. Greedy and plain
temperature sampling run on the device instead (sampling/device.py).
"""
from __future__ import annotations

from typing import Sequence

import numpy as np

from ..errors import OptionsError
from .options import Sampling

_MASK = (1 << 64) - 1


class SplitMix64:
    """sampling.rs:108-120."""

    def __init__(self, seed: int):
        self.state = seed & _MASK

    def uniform(self) -> float:
        self.state = (self.state + 0x9E3779B97F4A7C15) & _MASK
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
        z ^= z >> 31
        return (z >> 11) / float(1 << 53)


def sample_host(logits: np.ndarray, history: Sequence[int], rng: SplitMix64, options: Sampling) -> int:
    """One token id from one row of logits."""
    values = np.asarray(logits, dtype=np.float64)
    if values.size == 0 or not np.all(np.isfinite(values)):
        raise OptionsError("empty or non-finite logits")
    if options.greedy:
        return int(np.argmax(values))  # first maximum = lowest id on ties
    values = values.copy()
    if options.repeat_penalty != 1.0:
        seen = set()
        recent = list(history)[::-1][: options.repeat_last_n]
        for t in recent:
            if t not in seen:
                seen.add(t)
                if 0 <= t < values.size:
                    v = values[t]
                    values[t] = v * options.repeat_penalty if v <= 0.0 else v / options.repeat_penalty
    ids = np.arange(values.size)
    order = np.lexsort((ids, -values))  # value descending, then id ascending
    if 0 < options.top_k < values.size:
        order = order[: options.top_k]
    if options.temperature == 0.0:
        return int(order[0])
    kept = values[order]
    probs = np.exp((kept - kept[0]) / options.temperature)
    total = 0.0
    for p in probs:  # sequential sums, as the reference adds them
        total += p
    acc, keep = 0.0, len(order)
    for i, p in enumerate(probs):
        acc += p
        if acc / total >= options.top_p:
            keep = i + 1
            break
    order, probs = order[:keep], probs[:keep]
    total = 0.0
    for p in probs:
        total += p
    r = rng.uniform() * total
    acc = 0.0
    for token, p in zip(order, probs):
        acc += p
        if r < acc:
            return int(token)
    return int(order[-1])
