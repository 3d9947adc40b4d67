"""Which bfloat16 matrix-product kernel runs for a shape.

* up to 64 rows (decode): the weight-streaming kernel (csrc/gemm_bf16_stream.cu);
* otherwise, and for every shape the others refuse: the warp-level tiled kernel
  (csrc/gemm_bf16_mma.cu), which takes any M, N, K.
"""
from __future__ import annotations

import torch

from . import library
from .ops import _done, _ptr, _stream  # noqa: PLC2701  (same package)

force_tiled = False  # tests switch the streaming kernel off to compare both paths


def gemm_bf16(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, mode: int) -> None:
    """out (mode 0 bf16 store, 1 f32 store, 2 f32 add in place, 3 silu gate) = x . weight^T."""
    M, K = x.shape
    N = weight.shape[0]
    lib = library.load()
    if not force_tiled and lib.lrm_gemm_bf16_stream_supports(M, N, K) and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0:
        _done(lib.lrm_gemm_bf16_stream(_ptr(x), _ptr(weight), _ptr(out), M, N, K, mode, _stream()),
              "gemm_bf16_stream")
        return
    _done(lib.lrm_gemm_bf16_mma(_ptr(x), _ptr(weight), _ptr(out), M, N, K, mode, _stream()),
          "gemm_bf16_mma")
