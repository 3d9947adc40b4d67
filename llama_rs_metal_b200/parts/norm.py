"""RMSNorm."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from ..registry import register_norm
from ..weights.loader import TensorSpec
from .base import Norm


@register_norm("rms_norm")
class RMSNorm(Norm):
    """y = x / sqrt(mean(x^2) + eps) * w, statistics in float32
    (crates/metal-backend/src/shaders/elementwise.metal:31-46; no +1 offset for Llama)."""

    graph_safe = True
    folds_pending = True

    def __init__(self, size: int, eps: float):
        self.size = size
        self.eps = float(eps)
        self.weight: Optional[torch.Tensor] = None

    def tensors(self) -> Dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.size,))}

    def bind(self, weights, runtime) -> None:
        self.weight = weights["weight"].contiguous()

    def forward(self, hidden, ctx, rows=None):
        # partial sums a product left for the residual stream are added in the same pass
        pending = ctx.take_pending()
        return ops.rms_norm(hidden, self.weight, self.eps, ctx.runtime.dtype, rows=rows, partials=pending)
