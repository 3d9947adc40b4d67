"""Dense gated feed-forward."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..errors import UnsupportedError
from ..kernels import ops
from ..registry import register_feed_forward
from ..weights.loader import TensorSpec
from .base import FeedForward
from .linear import LinearWeight

GATE_BLOCK = 8  # rows of gate and up alternate in blocks of this many in the fused matrix


@register_feed_forward("gated_mlp")
class GatedMLP(FeedForward):
    """down( act(x Wg^T) * (x Wu^T) ), added to the residual stream
    (crates/model-runtime/src/execute.rs:251-267). Only SiLU is built, as in the
    reference (crates/model-format/src/mlx/config.rs:58-64)."""

    graph_safe = True

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "silu"):
        if activation != "silu":
            raise UnsupportedError("activation other than SiLU")
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.gate_up: Optional[LinearWeight] = None
        self.down: Optional[LinearWeight] = None
        self.block = GATE_BLOCK if intermediate_size % GATE_BLOCK == 0 else intermediate_size

    def tensors(self) -> Dict[str, TensorSpec]:
        h, i = self.hidden_size, self.intermediate_size
        return {"gate_proj.weight": TensorSpec((i, h)), "up_proj.weight": TensorSpec((i, h)),
                "down_proj.weight": TensorSpec((h, i))}

    def bind(self, weights, runtime) -> None:
        # Blocks of `block` gate rows alternate with the matching up rows, so a
        # product's epilogue finds both halves of a gated pair in one tile.
        g, u = weights["gate_proj.weight"], weights["up_proj.weight"]
        i, h, b = self.intermediate_size, self.hidden_size, self.block
        fused = torch.stack([g.reshape(i // b, b, h), u.reshape(i // b, b, h)], dim=1).reshape(2 * i, h)
        self.gate_up = LinearWeight(fused)
        self.down = LinearWeight(weights["down_proj.weight"])

    def forward(self, x, ctx, residual):
        if self.block == GATE_BLOCK and self.gate_up.supports_fused_gate(x.dtype):
            gated = self.gate_up(x, epilogue=ops.SILU_GATE)
        else:
            gated = ops.silu_mul(self.gate_up(x), self.block)
        return self.down(gated, epilogue=ops.ADD, out=residual, ctx=ctx)
