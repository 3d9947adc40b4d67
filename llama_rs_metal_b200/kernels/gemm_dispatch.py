"""Which bfloat16 matrix-product kernel runs for a shape.

* up to 16 rows (small decode batches): the weight-streaming kernel
  (csrc/gemm_bf16_stream.cu); it also takes 17-64 rows when the tensor-core kernel would
  leave most SMs idle and cannot split K (few output columns, epilogue other than "add");
* more rows (prompts, larger decode batches): the TMA + tcgen05 kernel
  (csrc/gemm_bf16_umma.cu), with 128 x 128 or 128 x 256 tiles, whichever needs less time by a
  count of rounds over the SMs and the measured cost of a tile; with at most 64 rows and few
  columns it cuts K into slices that meet by atomic adds in the float32 residual stream;
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
            names = {1: "a free stage", 2: "operand tiles", 3: "the accumulator", 4: "copies in flight",
                     5: "a free accumulator", 11: "the query tile", 12: "a key/value tile", 13: "scores",
                     14: "probabilities", 15: "weighted values", 16: "a free key/value stage"}
            kernel = "attention_prefill_umma" if code >= 11 else "gemm_bf16_umma"
            raise LlamaError(f"{kernel} gave up waiting for {names.get(code, code)}; its result is invalid")


def _wide(M: int, N: int) -> bool:
    if umma_width is not None:
        return umma_width == 256
    # Rounds of tiles over the SMs, times what a tile costs: a 128 x 256 tile has twice the work of
    # a 128 x 128 one but needs a third less operand traffic from L2 per product, which is what
    # bounds these kernels; measured, it costs about 1.4 narrow tiles.
    rows = -(-M // 128)
    narrow = -(-(rows * -(-N // 128)) // SM_COUNT)
    wide = 1.4 * -(-(rows * -(-N // 256)) // SM_COUNT)
    return wide <= narrow


STREAM_ROWS = 16  # up to this many rows the streaming kernel is the faster one
force_stream = False  # tests: keep 17-64 rows on the streaming kernel
stream_shape = None  # tests and tuning: (warps per CTA, K slices) of the streaming kernel instead of its own rule


def _few_rows_plan(M: int, N: int, K: int, mode: int):
    """For 17-64 rows: (use the tensor-core kernel?, K slices)."""
    tiles = -(-N // 128)
    if tiles >= SM_COUNT // 2:
        return True, 1
    if mode == 2:
        k_blocks = -(-K // 64)
        return True, max(1, min(k_blocks, 64, -(-SM_COUNT // tiles)))
    return False, 1


def gemm_bf16(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, mode: int) -> None:
    """out (mode 0 bf16 store, 1 f32 store, 2 f32 add in place, 3 silu gate) = x . weight^T."""
    global _status_dirty
    M, K = x.shape
    N = weight.shape[0]
    lib = library.load()
    aligned = x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0
    fast = not force_tiled and aligned
    stream_ok = fast and lib.lrm_gemm_bf16_stream_supports(M, N, K)
    umma_ok = fast and lib.lrm_gemm_bf16_umma_supports(M, N, K)
    wide, splits = _wide(M, N), 1
    if stream_ok and umma_ok and M > STREAM_ROWS and not force_stream:
        use_umma, splits = _few_rows_plan(M, N, K, mode)
        stream_ok = not use_umma
        wide = False if umma_width is None else wide
    if stream_ok:
        warps, slices = stream_shape if stream_shape is not None else (0, 0)
        _done(lib.lrm_gemm_bf16_stream_shaped(_ptr(x), _ptr(weight), _ptr(out), M, N, K, mode, warps,
                                              slices if mode == 2 else 0, _stream()), "gemm_bf16_stream")
        return
    if umma_ok:
        _status_dirty = True
        _done(lib.lrm_gemm_bf16_umma(_ptr(x), _ptr(weight), _ptr(out), M, N, K, mode,
                                     1 if wide else 0, splits, _ptr(_status_word(x.device)), _stream()),
              "gemm_bf16_umma")
        return
    _done(lib.lrm_gemm_bf16_mma(_ptr(x), _ptr(weight), _ptr(out), M, N, K, mode, _stream()),
          "gemm_bf16_mma")
