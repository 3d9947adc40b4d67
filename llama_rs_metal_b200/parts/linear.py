"""A stored [out, in] matrix and the product with it, shared by the parts that project."""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops


class LinearWeight:
    """y = x . W^T (no bias: crates/model-runtime/src/execute.rs:45-47).

    Precision follows storage: a matrix stored in bfloat16 multiplies bfloat16
    activations on the tensor cores; a matrix stored in 32-bit stays 32-bit and
    multiplies through the float32 kernel even under bfloat16 activations.
    """

    def __init__(self, weight: torch.Tensor):
        self.weight = weight.contiguous()

    @property
    def out_features(self) -> int:
        return self.weight.shape[0]

    def pick(self, x: torch.Tensor, temperature=None, seed: int = 0, keys=None):
        """The token chosen from each row's logits x . W^T (greedy, or temperature sampling with
        per-row keys), int32 [M], -1 for a row with a non-finite logit. The logits are not
        written where a kernel chooses in the product's epilogue."""
        if x.dtype == self.weight.dtype:
            ids = ops.linear_pick(x, self.weight, temperature, seed, keys)
            if ids is not None:
                return ids
        logits = self(x, out_dtype=torch.float32)
        if temperature is None:
            return ops.argmax_rows(logits)
        return ops.sample_gumbel_rows(logits, temperature, seed, keys)

    def supports_fused_gate(self, x_dtype: torch.dtype) -> bool:
        return self.weight.dtype == torch.bfloat16 and x_dtype == torch.bfloat16

    def __call__(self, x: torch.Tensor, epilogue: str = ops.STORE, out: Optional[torch.Tensor] = None,
                 out_dtype: Optional[torch.dtype] = None, ctx=None) -> torch.Tensor:
        """`ctx` (a StepContext) may be given with epilogue "add" for a part's last addition into
        the residual stream: while ctx.may_defer is set, a product that is cut into K slices
        leaves them in ctx.pending for the next norm to add instead of adding them here."""
        w = self.weight
        if x.dtype == w.dtype:
            if epilogue == ops.ADD and ctx is not None and ctx.may_defer:
                planes = ops.linear_slices(x, w)
                if planes is not None:
                    ctx.settle(out)  # at most one set of partial sums is pending at a time
                    ctx.pending = planes
                    return out
            return ops.linear(x, w, epilogue, out, out_dtype)
        if w.dtype == torch.float32 and x.dtype == torch.bfloat16:
            x32 = ops.cast(x, torch.float32)
            if epilogue == ops.ADD:
                return ops.linear(x32, w, ops.ADD, out)
            y = ops.linear(x32, w)
            return ops.cast(y, out_dtype or torch.bfloat16)
        # bfloat16 matrix under float32 activations does not occur: the float32
        # runtime widens every weight when it loads.
        return ops.linear(x, ops.cast(w, x.dtype), epilogue, out, out_dtype)
