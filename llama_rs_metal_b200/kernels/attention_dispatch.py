"""Which attention kernel runs for a geometry.

The row-wise kernel (csrc/attention_rowwise.cu) takes every head size up to
512, both dtypes, and is the only attention of the float32 path; tiled
bfloat16 kernels take over for the sizes they accept.
"""
from __future__ import annotations

import ctypes

import torch

from . import library
from .ops import _code, _done, _ptr, _stream  # noqa: PLC2701


def prefill(q, k, v, out, cu_seqlens, seq_of_token, max_seq_len: int, scale: float, window: int) -> None:
    T, Hq, d = q.shape
    lib = library.load()
    _done(lib.lrm_attention_packed_rowwise(_ptr(q), _ptr(k), _ptr(v), _ptr(out), _code(q.dtype),
                                           _ptr(cu_seqlens), _ptr(seq_of_token), T, Hq, k.shape[1], d,
                                           ctypes.c_float(scale), window, _stream()),
          "attention_packed_rowwise")


def decode(q, kv, out, slots, kv_lens, max_kv_len: int, scale: float, window: int) -> None:
    B, Hq, d = q.shape
    lib = library.load()
    _done(lib.lrm_attention_paged_rowwise(_ptr(q), _ptr(kv.k), _ptr(kv.v), _ptr(out), _code(q.dtype),
                                          _ptr(kv.page_table), kv.page_table.shape[1], _ptr(slots),
                                          _ptr(kv_lens), B, Hq, kv.kv_heads, d, kv.page_size,
                                          ctypes.c_float(scale), window, _stream()),
          "attention_paged_rowwise")
