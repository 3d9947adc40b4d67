"""Which bfloat16 matrix-product kernel runs for a shape.

The warp-level kernel (csrc/gemm_bf16_mma.cu) takes every shape and is the
fallback; faster kernels register themselves here with the shapes they accept.
"""
from __future__ import annotations

import torch

from . import library
from .ops import _done, _ptr, _stream  # noqa: PLC2701  (same package)


def gemm_bf16(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, mode: int) -> None:
    """out (mode 0 bf16 store, 1 f32 store, 2 f32 add in place, 3 silu gate) = x . weight^T."""
    M, K = x.shape
    N = weight.shape[0]
    lib = library.load()
    _done(lib.lrm_gemm_bf16_mma(_ptr(x), _ptr(weight), _ptr(out), M, N, K, mode, _stream()),
          "gemm_bf16_mma")
