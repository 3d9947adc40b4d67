"""Rotary position encoding (split-half or adjacent pairs) with linear and llama3 frequency scaling."""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch

from ..errors import InvalidError, UnsupportedError
from ..registry import register_position_encoding
from .base import PositionEncoding


_shared_frequencies = {}  # (device, frequencies) -> float32 tensor on that device

@register_position_encoding("rope")
class RotaryEmbedding(PositionEncoding):
    """angle(position, pair i) = position * scale * theta^(-2i/R) / factor[i]
    (crates/metal-backend/src/shaders/attention.metal:16-20). The per-pair
    inverse frequency is computed once on the host in double precision and
    rounded to float32; the kernel forms the angle as one float32 product.

    factor[i], llama3 rule (crates/model-format/src/mlx/config.rs:174-194):
    wavelen = 2 pi theta^(2i/R); below original/high -> 1; above original/low
    -> factor; between, smooth = (original/wavelen - low)/(high - low) and
    1/((1-smooth)/factor + smooth). `linear`: scale = 1/factor (config.rs:166-172).

    Pairing (attention.metal:14-16): split-half rotates dimension i with i + R/2; adjacent
    rotates 2i with 2i + 1 (config key rope_traditional). The kernels rotate split-half; for
    adjacent pairs the mixer reorders each head's query and key rows once (even dimensions of
    the rotary part first, then the odd ones), after which pair i is again (i, i + R/2) with
    the same frequency, and every score q.k is unchanged.
    """

    graph_safe = True

    def __init__(self, head_dim: int, rotary_dim: int, theta: float, scaling: str = "default",
                 factor: float = 1.0, low_freq_factor: float = 1.0, high_freq_factor: float = 4.0,
                 original_max_position_embeddings: int = 0, adjacent_pairs: bool = False):
        if rotary_dim <= 0 or rotary_dim > head_dim or rotary_dim % 2:
            raise InvalidError("rotary width must be even and at most the head size")
        if theta <= 0:
            raise InvalidError("rope theta must be positive")
        if scaling not in ("default", "linear", "llama3"):
            raise UnsupportedError(f"RoPE type {scaling}")
        self.head_dim, self.rotary_dim, self.theta = head_dim, rotary_dim, float(theta)
        self.scaling, self.factor = scaling, float(factor)
        self.low, self.high = float(low_freq_factor), float(high_freq_factor)
        self.original = int(original_max_position_embeddings)
        self.adjacent_pairs = bool(adjacent_pairs)
        self.inv_freq: Optional[torch.Tensor] = None

    def inverse_frequencies(self) -> List[float]:
        out = []
        R = self.rotary_dim
        for i in range(R // 2):
            freq = self.theta ** (-2.0 * i / R)
            if self.scaling == "linear":
                freq *= 1.0 / self.factor
            elif self.scaling == "llama3":
                wavelen = 2.0 * math.pi * self.theta ** (2.0 * i / R)
                if wavelen < self.original / self.high:
                    divisor = 1.0
                elif wavelen > self.original / self.low:
                    divisor = self.factor
                else:
                    smooth = (self.original / wavelen - self.low) / (self.high - self.low)
                    divisor = 1.0 / ((1.0 - smooth) / self.factor + smooth)
                freq /= divisor
            out.append(freq)
        return out

    def bind(self, weights, runtime) -> None:
        # layers with the same frequencies share one tensor, so that what is derived from it once
        # per step (a table of cosines and sines) serves them all
        frequencies = tuple(self.inverse_frequencies())
        key = (str(runtime.device), frequencies)
        if key not in _shared_frequencies:
            _shared_frequencies[key] = torch.tensor(frequencies, dtype=torch.float64) \
                .to(torch.float32).to(runtime.device)
        self.inv_freq = _shared_frequencies[key]

    def head_permutation(self) -> Optional[List[int]]:
        if not self.adjacent_pairs:
            return None
        R = self.rotary_dim
        return list(range(0, R, 2)) + list(range(1, R, 2)) + list(range(R, self.head_dim))

    def rotary_table(self) -> Optional[Tuple[torch.Tensor, int]]:
        return self.inv_freq, self.rotary_dim
