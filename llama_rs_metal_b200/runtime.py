"""What every part needs to know about where and how it computes."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .errors import UnsupportedError


@dataclass(frozen=True)
class Runtime:
    """Device and precision of one loaded model.

    dtype float32: weights, activations, cache and accumulation are all 32-bit
    (no tensor-core or reduced-precision mode). dtype bfloat16: weights as
    stored, bfloat16 activations and cache, float32 accumulation; the residual
    stream, norms, softmax and rotation angles stay float32 in both.
    """

    device: torch.device
    dtype: torch.dtype

    def __post_init__(self):
        if self.dtype not in (torch.float32, torch.bfloat16):
            raise UnsupportedError(f"dtype {self.dtype}: use float32 or bfloat16")

    @property
    def float32(self) -> bool:
        return self.dtype == torch.float32


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    table = {"float32": torch.float32, "fp32": torch.float32, "f32": torch.float32,
             "bfloat16": torch.bfloat16, "bf16": torch.bfloat16}
    try:
        return table[str(name).lower()]
    except KeyError:
        raise UnsupportedError(f"dtype {name!r}: use float32 or bfloat16") from None
