"""Python wrappers of the CUDA entry points.

Every wrapper checks devices, dtypes, contiguity and shapes on the host and
then launches on torch's current stream; memory comes from torch's allocator.
Nothing here computes on the CPU or calls a library model/attention routine.
A kernel that cannot take a size raises UnsupportedError with the reason.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from ..errors import InvalidError, KernelUnavailableError, UnsupportedError
from . import library

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}


def _code(dtype: torch.dtype) -> int:
    try:
        return _CODES[dtype]
    except KeyError:
        raise UnsupportedError(f"kernels take float32 or bfloat16, not {dtype}") from None


def _lib():
    return library.load()


def _stream() -> ctypes.c_void_p:
    # the raw handle of torch's current stream; the Stream object torch.cuda.current_stream()
    # builds costs several microseconds per launch, which a short prompt's ~150 launches feel
    return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(torch.cuda.current_device()))


def _ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _check(t: torch.Tensor, name: str, dtype=None, dims: Optional[int] = None) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelUnavailableError(f"{name} must be a CUDA tensor: there is no CPU path")
    if not t.is_contiguous():
        raise InvalidError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise InvalidError(f"{name} must be {dtype}, got {t.dtype}")
    if dims is not None and t.dim() != dims:
        raise InvalidError(f"{name} must have {dims} dimensions, got {tuple(t.shape)}")


_launches = 0


def launch_count() -> int:
    """How many kernels of this library have been launched (or captured) by this process."""
    return _launches


def _done(code: int, what: str, launches: int = 1) -> None:
    global _launches
    if code == 0:
        _launches += launches
        return
    if code == -1:
        raise InvalidError(f"{what}: bad argument")
    if code == -2:
        raise UnsupportedError(f"{what}: size not supported by this kernel")
    raise RuntimeError(f"{what}: CUDA error {code}")



ROW_RESERVE = 32  # rows an activation buffer holds at least (see _activation)


def _activation(rows: int, width: int, dtype: torch.dtype, device) -> torch.Tensor:
    """An uninitialised [rows, width] activation whose storage holds at least ROW_RESERVE rows: the
    tensor-core product may then name 32 rows in its tensor map of this operand, which TMA handles
    faster than fewer (the rows beyond `rows` only feed accumulator rows that are never stored)."""
    return torch.empty((max(rows, ROW_RESERVE), width), dtype=dtype, device=device)[:rows]


# --------------------------------------------------------------------------- embedding
def embed_rows(table: torch.Tensor, ids: torch.Tensor, scale: Optional[float] = None) -> torch.Tensor:
    """float32 [T, h] rows of `table` ([vocab, h], float32 or bfloat16) at int32 ids [T],
    multiplied by `scale` when one is given."""
    _check(table, "table", dims=2)
    _check(ids, "ids", torch.int32, 1)
    out = torch.empty((ids.numel(), table.shape[1]), dtype=torch.float32, device=table.device)
    _done(_lib().lrm_embed_rows(_ptr(table), _code(table.dtype), _ptr(ids), _ptr(out),
                                ids.numel(), table.shape[1], table.shape[0],
                                ctypes.c_float(1.0 if scale is None else scale), _stream()), "embed_rows")
    return out


# --------------------------------------------------------------------------- norm
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
             rows: Optional[torch.Tensor] = None, partials: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RMSNorm of float32 rows; see csrc/norm.cu for `rows` and `partials`."""
    _check(x, "x", torch.float32, 2)
    _check(weight, "weight", dims=1)
    hidden = x.shape[1]
    if weight.shape[0] != hidden:
        raise InvalidError(f"norm weight has {weight.shape[0]} elements, rows have {hidden}")
    n_rows = x.shape[0]
    if rows is not None:
        _check(rows, "rows", torch.int32, 1)
        n_rows = rows.numel()
    n_partials, stride = 0, 0
    if partials is not None:
        _check(partials, "partials", torch.float32, 3)
        if tuple(partials.shape[1:]) != tuple(x.shape):
            raise InvalidError("partials must be [n, T, h]")
        n_partials, stride = partials.shape[0], x.numel()
    out = _activation(n_rows, hidden, out_dtype, x.device)
    _done(_lib().lrm_rms_norm(_ptr(x), _ptr(weight), _code(weight.dtype), _ptr(out), _code(out_dtype),
                              _ptr(rows), _ptr(partials), n_partials, ctypes.c_longlong(stride),
                              n_rows, hidden, ctypes.c_float(eps), _stream()), "rms_norm")
    return out


# --------------------------------------------------------------------------- matrix products
STORE, ADD, SILU_GATE = "store", "add", "silu_gate"


def linear(x: torch.Tensor, weight: torch.Tensor, epilogue: str = STORE,
           out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """y = x . weight^T with weight [out, in] as stored.

    epilogue "store": returns [M, N] in `out_dtype` (default: x's dtype).
    epilogue "add":   adds into `out`, a float32 [M, N] tensor (the residual stream), in place.
    epilogue "silu_gate": weight rows alternate in blocks of 8 gate / 8 up rows;
                      returns silu(gate) * up as [M, N/2] (bfloat16 inputs only).
    float32 inputs run the true 32-bit kernel; bfloat16 inputs the tensor-core kernels.
    """
    _check(x, "x", dims=2)
    _check(weight, "weight", dims=2)
    M, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K:
        raise InvalidError(f"linear: x has {K} columns, weight has {weight.shape[1]}")
    if x.dtype != weight.dtype:
        raise InvalidError(f"linear: x is {x.dtype}, weight is {weight.dtype}")
    lib = _lib()
    if epilogue == ADD:
        if out is None:
            raise InvalidError("linear: epilogue 'add' needs the tensor to add into")
        _check(out, "out", torch.float32, 2)
        if tuple(out.shape) != (M, N):
            raise InvalidError(f"linear: out must be [{M}, {N}]")
    if x.dtype == torch.float32:
        if epilogue == SILU_GATE:
            raise UnsupportedError("linear: the float32 kernel has no fused gate epilogue")
        if epilogue == STORE:
            if out_dtype not in (None, torch.float32):
                raise InvalidError("linear: float32 inputs give float32 outputs")
            out = torch.empty((M, N), dtype=torch.float32, device=x.device)
        _done(lib.lrm_gemm_f32(_ptr(x), _ptr(weight), _ptr(out), M, N, K,
                               1 if epilogue == ADD else 0, _stream()), "gemm_f32")
        return out
    if x.dtype != torch.bfloat16:
        raise UnsupportedError(f"linear: dtype {x.dtype}")
    if epilogue == STORE:
        out_dtype = out_dtype or torch.bfloat16
        out = _activation(M, N, out_dtype, x.device)
        mode = 0 if out_dtype == torch.bfloat16 else 1
        if out_dtype not in (torch.bfloat16, torch.float32):
            raise UnsupportedError(f"linear: out dtype {out_dtype}")
    elif epilogue == ADD:
        mode = 2
    elif epilogue == SILU_GATE:
        if N % 16 != 0:
            raise UnsupportedError("linear: the fused gate epilogue needs a multiple of 16 rows")
        out = _activation(M, N // 2, torch.bfloat16, x.device)
        mode = 3
    else:
        raise InvalidError(f"linear: unknown epilogue {epilogue!r}")
    from . import gemm_dispatch
    gemm_dispatch.gemm_bf16(x, weight, out, mode)
    return out


def linear_slices(x: torch.Tensor, weight: torch.Tensor) -> Optional[torch.Tensor]:
    """x . weight^T as float32 partial products over K slices [slices, M, N] (their sum in plane
    order is the product), or None when this product is not cut. Only narrow bfloat16 products
    are cut; rms_norm(partials=...) or add_planes_ adds the planes to the residual stream."""
    _check(x, "x", dims=2)
    _check(weight, "weight", dims=2)
    if weight.shape[1] != x.shape[1]:
        raise InvalidError(f"linear: x has {x.shape[1]} columns, weight has {weight.shape[1]}")
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        return None
    from . import gemm_dispatch
    return gemm_dispatch.gemm_bf16_slices(x, weight)


def add_planes_(x: torch.Tensor, planes: torch.Tensor) -> torch.Tensor:
    """x += planes[0] + planes[1] + ... (in that order); x float32, planes [n, *x.shape] float32."""
    _check(x, "x", torch.float32)
    _check(planes, "planes", torch.float32)
    if tuple(planes.shape[1:]) != tuple(x.shape):
        raise InvalidError(f"add_planes_: planes {tuple(planes.shape)} do not match {tuple(x.shape)}")
    _done(_lib().lrm_add_planes(_ptr(x), _ptr(planes), planes.shape[0], ctypes.c_longlong(x.numel()),
                                _stream()), "add_planes_")
    return x


def scale_(x: torch.Tensor, factor: float) -> torch.Tensor:
    """x *= factor in place (float32)."""
    _check(x, "x", torch.float32)
    _done(_lib().lrm_scale_inplace(_ptr(x), ctypes.c_float(factor), ctypes.c_longlong(x.numel()), _stream()),
          "scale_")
    return x


def silu_mul(gate_up: torch.Tensor, block: int) -> torch.Tensor:
    """silu(gate) * up from [T, 2I] whose columns alternate in blocks of `block` gate / up."""
    _check(gate_up, "gate_up", dims=2)
    inter = gate_up.shape[1] // 2
    if gate_up.shape[1] % 2 or inter % block:
        raise InvalidError("silu_mul: width must be 2*I with I a multiple of the block")
    out = _activation(gate_up.shape[0], inter, gate_up.dtype, gate_up.device)
    _done(_lib().lrm_silu_mul(_ptr(gate_up), _ptr(out), _code(gate_up.dtype),
                              ctypes.c_longlong(gate_up.shape[0]), inter, block, _stream()), "silu_mul")
    return out


def add_(x: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    """x += delta, x float32 (the residual sum is always 32-bit)."""
    _check(x, "x", torch.float32)
    _check(delta, "delta")
    if x.shape != delta.shape:
        raise InvalidError(f"add_: shapes {tuple(x.shape)} and {tuple(delta.shape)}")
    _done(_lib().lrm_add_inplace(_ptr(x), _ptr(delta), _code(delta.dtype),
                                 ctypes.c_longlong(x.numel()), _stream()), "add_")
    return x


def cast(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    _check(x, "x")
    if x.dtype == dtype:
        return x
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    _done(_lib().lrm_cast(_ptr(x), _code(x.dtype), _ptr(out), _code(dtype),
                          ctypes.c_longlong(x.numel()), _stream()), "cast")
    return out


# --------------------------------------------------------------------------- rope + cache store
def rope_store(qkv: torch.Tensor, q_heads: int, kv_heads: int, head_dim: int,
               inv_freq: Optional[torch.Tensor], rotary: int, positions: torch.Tensor,
               kv=None, dest_rows: Optional[torch.Tensor] = None,
               keep_packed: bool = True) -> Tuple[torch.Tensor, Optional[torch.Tensor], Optional[torch.Tensor]]:
    """Rotate q and k of a fused [T, (Hq+2Hk)*d] projection and store k, v.

    Returns (q [T,Hq,d], k [T,Hk,d] or None, v [T,Hk,d] or None); k and v are
    returned when `keep_packed`, and written to the paged cache view `kv` at
    `dest_rows` (int32 [T]: page * page_size + row, < 0 = not stored) when given.
    """
    _check(qkv, "qkv", dims=2)
    T = qkv.shape[0]
    if qkv.shape[1] != (q_heads + 2 * kv_heads) * head_dim:
        raise InvalidError("rope_store: qkv width does not match the head geometry")
    if head_dim % 2:
        raise UnsupportedError("rope_store: head size must be even")
    _check(positions, "positions", torch.int32, 1)
    if inv_freq is not None:
        _check(inv_freq, "inv_freq", torch.float32, 1)
        if inv_freq.numel() != rotary // 2:
            raise InvalidError("rope_store: inv_freq must have rotary/2 entries")
    dev = qkv.device
    q = torch.empty((T, q_heads, head_dim), dtype=qkv.dtype, device=dev)
    k = torch.empty((T, kv_heads, head_dim), dtype=qkv.dtype, device=dev) if keep_packed else None
    v = torch.empty((T, kv_heads, head_dim), dtype=qkv.dtype, device=dev) if keep_packed else None
    k_pages = v_pages = None
    page_size = 1
    if kv is not None:
        k_pages, v_pages, page_size = kv.k, kv.v, kv.page_size
        _check(k_pages, "k pages", qkv.dtype, 4)
        _check(v_pages, "v pages", qkv.dtype, 4)
        _check(dest_rows, "dest_rows", torch.int32, 1)
        if dest_rows.numel() != T:
            raise InvalidError("rope_store: one destination row per token")
        if tuple(k_pages.shape[1:]) != (kv_heads, page_size, head_dim):
            raise InvalidError("rope_store: cache pages do not match the head geometry")
    _done(_lib().lrm_rope_store(_ptr(qkv), _code(qkv.dtype), _ptr(q), _ptr(k), _ptr(v),
                                _ptr(k_pages), _ptr(v_pages), _ptr(dest_rows if kv is not None else None),
                                _ptr(positions), _ptr(inv_freq), rotary, T, q_heads,
                                kv_heads, head_dim, page_size, _stream()), "rope_store")
    return q, k, v


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """float32 [T, R/2, 2]: (cos, sin) of float32(position) * inv_freq, the angles rope_store forms."""
    _check(positions, "positions", torch.int32, 1)
    _check(inv_freq, "inv_freq", torch.float32, 1)
    T, half = positions.numel(), inv_freq.numel()
    table = torch.empty((T, half, 2), dtype=torch.float32, device=positions.device)
    _done(_lib().lrm_rope_table(_ptr(positions), _ptr(inv_freq), _ptr(table), T, half, _stream()), "rope_table")
    return table


def linear_rope_store(x: torch.Tensor, weight: torch.Tensor, q_heads: int, kv_heads: int, head_dim: int,
                      table: Optional[torch.Tensor], kv=None, dest_rows: Optional[torch.Tensor] = None):
    """rope_store(linear(x, weight)) for a prompt in one launch where the tensor-core product takes
    the shape: (q [T,Hq,d], k [T,Hk,d], v [T,Hk,d]), with k and v also written to the cache view
    `kv` at `dest_rows`; None where it does not (nothing was launched). `table` from rope_table
    (rotation of the whole head) or None (no rotation). Bit-equal to the two separate kernels."""
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or x.dim() != 2:
        return None
    T = x.shape[0]
    if table is not None and tuple(table.shape) != (T, head_dim // 2, 2):
        return None
    if kv is not None and (kv.k.dtype != torch.bfloat16 or tuple(kv.k.shape[1:]) != (kv_heads, kv.page_size, head_dim)):
        return None
    q = torch.empty((T, q_heads, head_dim), dtype=x.dtype, device=x.device)
    k = torch.empty((T, kv_heads, head_dim), dtype=x.dtype, device=x.device)
    v = torch.empty((T, kv_heads, head_dim), dtype=x.dtype, device=x.device)
    from . import gemm_dispatch
    if not gemm_dispatch.gemm_bf16_qkv(x, weight, q, k, v, kv, dest_rows, table):
        return None
    return q, k, v


# --------------------------------------------------------------------------- attention
def attention_prefill(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: torch.Tensor,
                      seq_of_token: torch.Tensor, max_seq_len: int, scale: float,
                      window: Optional[int] = None) -> torch.Tensor:
    """Causal GQA over the step's own packed k, v (sequences start at position 0). -> [T, Hq*d]"""
    _check(q, "q", dims=3)
    _check(k, "k", q.dtype, 3)
    _check(v, "v", q.dtype, 3)
    _check(cu_seqlens, "cu_seqlens", torch.int32, 1)
    _check(seq_of_token, "seq_of_token", torch.int32, 1)
    T, Hq, d = q.shape
    Hk = k.shape[1]
    if k.shape != v.shape or k.shape[0] != T or k.shape[2] != d or Hq % Hk:
        raise InvalidError("attention_prefill: q, k, v shapes do not agree")
    out = _activation(T, Hq * d, q.dtype, q.device)
    from . import attention_dispatch
    attention_dispatch.prefill(q, k, v, out, cu_seqlens, seq_of_token, max_seq_len, scale, window or 0)
    return out


def attention_decode(q: torch.Tensor, kv, slots: torch.Tensor, kv_lens: torch.Tensor,
                     max_kv_len: int, scale: float, window: Optional[int] = None) -> torch.Tensor:
    """One query per sequence over its cached keys (the newest already stored). -> [B, Hq*d]"""
    _check(q, "q", dims=3)
    _check(kv.k, "k pages", q.dtype, 4)
    _check(kv.v, "v pages", q.dtype, 4)
    _check(kv.page_table, "page table", torch.int32, 2)
    _check(slots, "slots", torch.int32, 1)
    _check(kv_lens, "kv_lens", torch.int32, 1)
    B, Hq, d = q.shape
    if tuple(kv.k.shape[1:]) != (kv.kv_heads, kv.page_size, d) or Hq % kv.kv_heads:
        raise InvalidError("attention_decode: cache pages do not match the query geometry")
    out = _activation(B, Hq * d, q.dtype, q.device)
    from . import attention_dispatch
    attention_dispatch.decode(q, kv, out, slots, kv_lens, max_kv_len, scale, window or 0)
    return out


def attention_extend(q: torch.Tensor, kv, cu_seqlens: torch.Tensor, seq_of_token: torch.Tensor,
                     positions: torch.Tensor, slots: torch.Tensor, kv_lens: torch.Tensor, max_seq_len: int,
                     scale: float, window: Optional[int] = None) -> torch.Tensor:
    """Several queries per sequence over the cache, which already holds the step's own keys:
    query t (packed, of sequence seq_of_token[t]) sees the keys up to positions[t]. -> [T, Hq*d]"""
    _check(q, "q", dims=3)
    _check(kv.k, "k pages", q.dtype, 4)
    _check(kv.v, "v pages", q.dtype, 4)
    _check(kv.page_table, "page table", torch.int32, 2)
    T, Hq, d = q.shape
    for name, t, n in (("cu_seqlens", cu_seqlens, None), ("seq_of_token", seq_of_token, T),
                       ("positions", positions, T), ("slots", slots, cu_seqlens.numel() - 1),
                       ("kv_lens", kv_lens, cu_seqlens.numel() - 1)):
        _check(t, name, torch.int32, 1)
        if n is not None and t.numel() != n:
            raise InvalidError(f"attention_extend: {name} must have {n} entries")
    if tuple(kv.k.shape[1:]) != (kv.kv_heads, kv.page_size, d) or Hq % kv.kv_heads:
        raise InvalidError("attention_extend: cache pages do not match the query geometry")
    out = _activation(T, Hq * d, q.dtype, q.device)
    from . import attention_dispatch
    attention_dispatch.extend(q, kv, out, cu_seqlens, seq_of_token, positions, slots, kv_lens, max_seq_len,
                              scale, window or 0)
    return out


def attention_decode_fused_supported(dtype, head_dim: int, page_size: int, rotary: int, window) -> bool:
    from . import attention_dispatch
    return attention_dispatch.decode_fused_supported(dtype, head_dim, page_size, rotary, window)


def attention_decode_prefers_fused(seqs: int, kv_heads: int, group: int, head_dim: int, max_kv_len: int) -> bool:
    """Whether the one-launch kernel is expected to beat the separate kernels for this step's geometry."""
    from . import attention_dispatch
    return attention_dispatch.decode_prefers_fused(seqs, kv_heads, group, head_dim, max_kv_len)


def attention_decode_fused(qkv: torch.Tensor, q_heads: int, inv_freq: Optional[torch.Tensor], rotary: int,
                           positions: torch.Tensor, kv, dest_rows: torch.Tensor, slots: torch.Tensor,
                           kv_lens: torch.Tensor, max_kv_len: int, scale: float,
                           order: Optional[torch.Tensor] = None, fill: int = 4) -> torch.Tensor:
    """A decode step's attention from its fused, unrotated [B, (Hq+2Hk)*d] projection: rotates q and
    the new k, stores the new k and v at `dest_rows`, attends over the cache (kv_lens counts the new
    token) and merges the splits, in one launch. -> [B, Hq*d]. `order` (int32 [B], made on the host and
    copied before the step, because the kernel reads it before it waits for the kernels ahead of
    it): the sequences' work is handed out in this order, longest first when lengths are unequal;
    `fill`: their mean length in quarters of the longest (launch geometry only)."""
    _check(qkv, "qkv", torch.bfloat16, 2)
    d, Hk = kv.head_dim, kv.kv_heads
    if qkv.shape[1] != (q_heads + 2 * Hk) * d or q_heads % Hk:
        raise InvalidError("attention_decode_fused: qkv width does not match the head geometry")
    _check(kv.k, "k pages", qkv.dtype, 4)
    _check(kv.v, "v pages", qkv.dtype, 4)
    if tuple(kv.k.shape[1:]) != (Hk, kv.page_size, d):
        raise InvalidError("attention_decode_fused: cache pages do not match the head geometry")
    _check(kv.page_table, "page table", torch.int32, 2)
    B = qkv.shape[0]
    for name, t in (("positions", positions), ("dest_rows", dest_rows), ("slots", slots), ("kv_lens", kv_lens)):
        _check(t, name, torch.int32, 1)
        if t.numel() != B:
            raise InvalidError(f"attention_decode_fused: one entry of {name} per sequence")
    if inv_freq is not None:
        _check(inv_freq, "inv_freq", torch.float32, 1)
        if inv_freq.numel() != rotary // 2:
            raise InvalidError("attention_decode_fused: inv_freq must have rotary/2 entries")
    else:
        rotary = 0
    if not attention_decode_fused_supported(qkv.dtype, d, kv.page_size, rotary, kv.window):
        raise UnsupportedError("attention_decode_fused: geometry not supported; use rope_store and attention_decode")
    out = _activation(B, q_heads * d, qkv.dtype, qkv.device)
    from . import attention_dispatch
    if order is not None:
        _check(order, "order", torch.int32, 1)
        if order.numel() != B:
            raise InvalidError("attention_decode_fused: one entry of order per sequence")
    attention_dispatch.decode_fused(qkv, positions, inv_freq, rotary, kv, dest_rows, out, slots, kv_lens,
                                    max_kv_len, q_heads, scale, order, fill)
    return out


def attend(projected: torch.Tensor, **geometry) -> torch.Tensor:
    """A layer's attention for one step from its projection (see attention_dispatch.attend)."""
    from . import attention_dispatch
    return attention_dispatch.attend(projected, **geometry)


# --------------------------------------------------------------------------- sampling
def _pick_scratch(logits: torch.Tensor):
    pieces = _lib().lrm_pick_pieces(logits.shape[1])
    values = torch.empty((logits.shape[0], pieces), dtype=torch.float32, device=logits.device)
    ids = torch.empty((logits.shape[0], pieces), dtype=torch.int32, device=logits.device)
    return values, ids


PICK_ROWS = 12  # up to this many rows the streaming product is the head's fastest kernel, and it can choose

_pick_words_by_device = {}


def _pick_words(device: torch.device) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per device: 64 running-best words and 64 flags for the head product that chooses in its
    epilogue. Zero between calls (the kernel that reads the winners clears them), so every call
    on a stream can share them; reset_pick_scratch() zeroes them after a failed step."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index not in _pick_words_by_device:
        _pick_words_by_device[index] = (torch.zeros(64, dtype=torch.int64, device=device),
                                        torch.zeros(64, dtype=torch.int32, device=device))
    return _pick_words_by_device[index]


def reset_pick_scratch() -> None:
    for best, bad in _pick_words_by_device.values():
        best.zero_()
        bad.zero_()


def linear_pick(x: torch.Tensor, weight: torch.Tensor, temperature: Optional[float] = None, seed: int = 0,
                keys: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """int32 [M]: the token chosen from the logits x . weight^T of each row, without writing the
    logits: every CTA of the head product offers its best (score, id) per row to the row's
    running best with an atomic maximum, and a second small kernel reads the winners.
    temperature None: greedy, as argmax_rows; else a draw from softmax(logits / temperature) with
    the noise of sample_gumbel_rows for the same seed and keys (int64 [M]). -1 marks a row with a
    non-finite logit. None when no kernel takes this product that way (float32, more rows than
    the streaming product is the fastest for, unaligned): the caller then writes the logits and
    picks from them."""
    _check(x, "x", dims=2)
    _check(weight, "weight", dims=2)
    M, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K:
        raise InvalidError(f"linear_pick: x has {K} columns, weight has {weight.shape[1]}")
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or M > PICK_ROWS:
        return None
    lib = _lib()
    if not lib.lrm_gemm_bf16_stream_supports(M, N, K) or x.data_ptr() % 16 or weight.data_ptr() % 16:
        return None
    if temperature is not None:
        if keys is None or not temperature > 0:
            raise InvalidError("linear_pick: temperature sampling needs a positive temperature and one key per row")
        _check(keys, "keys", torch.int64, 1)
        if keys.numel() != M:
            raise InvalidError("linear_pick: one key per row")
    best, bad = _pick_words(x.device)
    out = torch.empty((M,), dtype=torch.int32, device=x.device)
    _done(lib.lrm_gemm_bf16_stream_pick(_ptr(x), _ptr(weight), M, N, K, _ptr(best), _ptr(bad), _ptr(out),
                                        ctypes.c_float(temperature if temperature is not None else 1.0),
                                        ctypes.c_ulonglong(seed & ((1 << 64) - 1)),
                                        _ptr(keys if temperature is not None else None), _stream()),
          "gemm_bf16_stream_pick", launches=2)
    return out


def argmax_rows(logits: torch.Tensor) -> torch.Tensor:
    """int32 [n]: largest logit per row, lowest id on ties, -1 for a row with a non-finite logit."""
    _check(logits, "logits", torch.float32, 2)
    out = torch.empty((logits.shape[0],), dtype=torch.int32, device=logits.device)
    values, ids = _pick_scratch(logits)
    _done(_lib().lrm_argmax_rows(_ptr(logits), _ptr(out), _ptr(values), _ptr(ids), logits.shape[0],
                                 logits.shape[1], _stream()), "argmax_rows", launches=2)
    return out


def sample_gumbel_rows(logits: torch.Tensor, temperature: float, seed: int, keys: torch.Tensor) -> torch.Tensor:
    """int32 [n]: a draw from softmax(logits / temperature) per row; `keys` int64 [n] names each row's stream."""
    _check(logits, "logits", torch.float32, 2)
    _check(keys, "keys", torch.int64, 1)
    if keys.numel() != logits.shape[0]:
        raise InvalidError("sample_gumbel_rows: one key per row")
    if not temperature > 0:
        raise InvalidError("sample_gumbel_rows: temperature must be positive")
    out = torch.empty((logits.shape[0],), dtype=torch.int32, device=logits.device)
    values, ids = _pick_scratch(logits)
    _done(_lib().lrm_sample_gumbel_rows(_ptr(logits), _ptr(out), _ptr(values), _ptr(ids), logits.shape[0],
                                        logits.shape[1], ctypes.c_float(temperature),
                                        ctypes.c_ulonglong(seed & ((1 << 64) - 1)), _ptr(keys),
                                        _stream()), "sample_gumbel_rows", launches=2)
    return out
