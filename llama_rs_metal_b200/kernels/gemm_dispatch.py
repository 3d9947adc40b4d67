"""Which bfloat16 matrix-product kernel runs for a shape.

* up to 64 rows (decode): the weight-streaming kernel (csrc/gemm_bf16_stream.cu);
* more rows (prompts): the TMA + tcgen05 kernel (csrc/gemm_bf16_umma.cu), with
  128 x 128 or 128 x 256 tiles, whichever leaves fewer idle SMs in the last wave;
* every shape the others refuse (K not a multiple of 8, unaligned views): the
  warp-level tiled kernel (csrc/gemm_bf16_mma.cu), which takes any M, N, K.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..errors import LlamaError
from . import library
from .ops import _done, _ptr, _stream  # noqa: PLC2701  (same package)

SM_COUNT = 148
force_tiled = False  # tests switch the fast kernels off to compare both paths
umma_width: Optional[int] = None  # tests pin the tile width (128 or 256)

_status: Dict[int, torch.Tensor] = {}
_status_dirty = False


def _status_word(device: torch.device) -> torch.Tensor:
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index not in _status:
        _status[index] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[index]


def check_status() -> None:
    """Raise if a tensor-core kernel gave up on a wait since the last check (reads 4 bytes back)."""
    global _status_dirty
    if not _status_dirty:
        return
    _status_dirty = False
    for word in _status.values():
        code = int(word.item())
        if code != 0:
            word.zero_()
            names = {1: "a free stage", 2: "operand tiles", 3: "the accumulator", 4: "copies in flight"}
            raise LlamaError(f"gemm_bf16_umma gave up waiting for {names.get(code, code)}; its result is invalid")


def _wide(M: int, N: int) -> bool:
    if umma_width is not None:
        return umma_width == 256
    rows = -(-M // 128)
    narrow = -(-(rows * -(-N // 128)) // SM_COUNT)
    wide = 2 * -(-(rows * -(-N // 256)) // SM_COUNT)
    return wide <= narrow


def gemm_bf16(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, mode: int) -> None:
    """out (mode 0 bf16 store, 1 f32 store, 2 f32 add in place, 3 silu gate) = x . weight^T."""
    global _status_dirty
    M, K = x.shape
    N = weight.shape[0]
    lib = library.load()
    aligned = x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0
    if not force_tiled and aligned and lib.lrm_gemm_bf16_stream_supports(M, N, K):
        _done(lib.lrm_gemm_bf16_stream(_ptr(x), _ptr(weight), _ptr(out), M, N, K, mode, _stream()),
              "gemm_bf16_stream")
        return
    if not force_tiled and aligned and lib.lrm_gemm_bf16_umma_supports(M, N, K):
        _status_dirty = True
        _done(lib.lrm_gemm_bf16_umma(_ptr(x), _ptr(weight), _ptr(out), M, N, K, mode,
                                     1 if _wide(M, N) else 0, _ptr(_status_word(x.device)), _stream()),
              "gemm_bf16_umma")
        return
    _done(lib.lrm_gemm_bf16_mma(_ptr(x), _ptr(weight), _ptr(out), M, N, K, mode, _stream()),
          "gemm_bf16_mma")
