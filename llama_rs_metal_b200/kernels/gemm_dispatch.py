"""Which bfloat16 matrix-product kernel runs for a shape.

* up to 8 rows (small decode batches): the weight-streaming kernel
  (csrc/gemm_bf16_stream.cu); it also takes 9-64 rows when the tensor-core kernel would
  leave most SMs idle and cannot split K (few output columns, epilogue other than "add");
* more rows (prompts, larger decode batches): the TMA + tcgen05 kernel
  (csrc/gemm_bf16_umma.cu), with 128 x 128, 128 x 256 or 256 x 256 tiles, whichever needs less
  time by a count of rounds over the SMs and the measured cost of a tile;
* a narrow product that is to be added to the residual stream may be cut into K slices so that
  every SM works: the slices are stored as planes of an [slices, M, N] tensor, which the next
  norm adds in slice order (gemm_bf16_slices); nothing meets by atomics, so the same step gives
  the same bits every time;
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
umma_width: Optional[int] = None  # tests pin the tile: 128 (128 x 128), 256 (128 x 256), 512 (256 x 256), 192 (128 x 192)

_status: Dict[int, torch.Tensor] = {}
_status_dirty = False
_status_launches = 0  # launches (or captures) so far of kernels that write the status word


def mark_status_dirty() -> None:
    """A kernel with bounded waits was launched (directly, or by replaying a CUDA graph that holds
    one): the next check_status() reads the status word."""
    global _status_dirty, _status_launches
    _status_dirty = True
    _status_launches += 1


def status_launch_count() -> int:
    return _status_launches


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
                     14: "probabilities", 15: "weighted values", 16: "a free key/value stage",
                     17: "aligned shared memory", 21: "the query tiles", 22: "a key/value tile", 23: "scores",
                     24: "probabilities", 25: "the output", 26: "a free key/value stage", 27: "aligned shared memory"}
            names.update({31: "a free stage", 32: "operand tiles", 33: "the accumulator", 34: "copies in flight",
                          35: "a free accumulator"})
            kernel = "gemm_bf16_umma_pair" if code >= 31 else "attention_prefill_pingpong" if code >= 21 else \
                "attention_prefill_umma" if code >= 11 else "gemm_bf16_umma"
            raise LlamaError(f"{kernel} gave up waiting for {names.get(code, code)}; its result is invalid")


# What an output tile costs relative to a 128 x 128 one. Operand traffic from L2 bounds these
# products (measured: the tensor pipe is busy 38-44 % of the time with 128 x 128 tiles, 66-71 %
# with 128 x 256), so a larger tile does more work per byte. A 256 x 256 tile fills the tensor
# memory, so its epilogue does not run under the next tile's MMAs: it pays only when K is long
# (measured at 8,192 rows: 0.85 of the 128 x 256 time at K = 8192, 1.05 at K = 2048 with a plain
# epilogue, 1.3 with the SiLU gate).
def _tile_costs(K: int, mode: int):
    k_blocks = max(1, -(-K // 64))
    epilogue = 1.1 if mode == 3 else 0.55
    return ((128, 128, 1.0), (128, 256, 1.4), (256, 256, 1.4 * (1.55 + epilogue * 32 / k_blocks)), (128, 192, 1.2))


PAIR = 4  # tile code of the kernel that runs a 256 x 256 tile on two SMs


def _pair_cost(K: int, rounds: int) -> float:
    """`rounds` rounds of 256 x 256 tiles over the pairs of SMs, in units of a 128 x 128 tile on one
    SM: each SM does a 128 x 256 tile's work with a third less operand traffic and a hidden
    epilogue (measured at 2,048 rows: gate/up 104 us against 115, down 60 against 64, the 8B shape's
    QKV 88 against 97; at 4,096 rows 5-15 % faster than the best single-SM tile throughout); its
    start-up (a cluster to place, tensor memory allocated by both CTAs together) weighs more the
    shorter K is."""
    return 1.27 * rounds + 0.2 * 32 / max(1, -(-K // 64))


_pair_room = {}


def pair_room() -> int:
    """Pairs of SMs the two-CTA product can occupy at once (0: not on this device)."""
    device = torch.cuda.current_device()
    if device not in _pair_room:
        _pair_room[device] = 0 if force_tiled else int(library.load().lrm_gemm_bf16_umma_pair_room())
    return _pair_room[device]


def tile_choice(M: int, N: int, K: int = 2048, mode: int = 0, pairs: int = 0, multiple_of: int = 1) -> int:
    """0: 128 x 128, 1: 128 x 256, 2: 256 x 256, 3: 128 x 192 output tiles on one SM each, or 4: 256 x
    256 tiles on `pairs` pairs of SMs (0: not to be had): least rounds over the SMs times cost, among
    the tiles whose width is a multiple of `multiple_of` (an epilogue that works on whole heads)."""
    if umma_width is not None and {128: 128, 256: 256, 512: 256, 192: 192, "pair": 256}[umma_width] % multiple_of == 0:
        return {128: 0, 256: 1, 512: 2, 192: 3, "pair": PAIR}[umma_width]
    best, best_cost = 0, None
    for index, (rows, columns, cost) in enumerate(_tile_costs(K, mode)):
        if columns % multiple_of or (pairs > 0 and index == 2):  # a pair does what the 256 x 256 tile does, better
            continue
        rounds = -(-(-(-M // rows) * -(-N // columns)) // SM_COUNT)
        if best_cost is None or rounds * cost < best_cost:
            best, best_cost = index, rounds * cost
    if pairs > 0 and mode <= 3:
        rounds = -(-(-(-M // 256) * -(-N // 256)) // pairs)
        if _pair_cost(K, rounds) < best_cost:
            best = PAIR
    return best


def _wide(M: int, N: int) -> bool:
    return tile_choice(M, N) >= 1


STREAM_ROWS = 8  # up to this many rows the streaming kernel is always the faster one
force_stream = False  # tests: keep 17-64 rows on the streaming kernel
stream_shape = None  # tests and tuning: (warps per CTA, K slices) of the streaming kernel instead of its own rule


def _few_rows_plan(M: int, N: int, K: int, mode: int):
    """For 9-64 rows: (use the tensor-core kernel?, K slices). Measured at the 1B layer sizes:
    many column tiles run as they are from 13 rows on; a product whose slices the next norm adds
    (mode 4) is cut into as many K slices as keep every item in one round over the SMs, except a
    small one (8 MB of weights, up to 32 rows), which the streaming kernel does faster; the rest
    streams."""
    tiles = -(-N // 128)
    if tiles >= SM_COUNT // 2:
        return M > 12, 1
    if mode == 4:
        if M <= 32 and N * K <= 4 * 1024 * 1024:
            return False, 1
        k_blocks = -(-K // 64)
        return True, max(1, min(k_blocks, 64, SM_COUNT // tiles))
    return False, 1


def _fast_kernels(x: torch.Tensor, weight: torch.Tensor, lib):
    M, K = x.shape
    N = weight.shape[0]
    aligned = x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0
    fast = not force_tiled and aligned
    return (fast and bool(lib.lrm_gemm_bf16_stream_supports(M, N, K)),
            fast and bool(lib.lrm_gemm_bf16_umma_supports(M, N, K)))


def _sliced_plan(M: int, N: int, K: int):
    """(tile, K slices) for a product of a few hundred rows that goes into the residual stream as
    planes: 128 x 128 or 128 x 256 tiles, K cut until the items fill the SMs once (no slice shorter
    than 256), whichever is estimated faster, or (0, 1) where the uncut product added in place is.
    Measured per 64 of K and item: 0.30 us with 128 x 128 tiles, 0.35 us with 128 x 256 (twice the
    work), more where few row tiles share a W tile that comes from HBM; a plane more costs its write
    and the norm's read of it, and the norm adds planes eight at a time. Whole prompt steps of the
    1B shape, this rule against 128 x 128 tiles only: 768 tokens 2.46 against 2.69 ms, 1,024 tokens
    2.92 against 3.03, 128 tokens 1.39 against 1.41, 256 and 512 tokens unchanged."""
    k_blocks = -(-K // 64)
    best, whole = None, None
    row_tiles = -(-M // 128)
    for tile, (columns, per_block) in enumerate(((128, 0.30), (256, 0.35))):
        # with few row tiles a W tile is fetched from HBM for almost every item: 44 GB/s per SM
        per_block = max(per_block, columns * 128 / 44e3 / row_tiles)
        tiles = row_tiles * -(-N // columns)
        uncut = -(-tiles // SM_COUNT) * k_blocks * per_block       # added in place, no planes
        whole = uncut if whole is None else min(whole, uncut)
        fill = max(1, min(k_blocks // 4, SM_COUNT // tiles))
        for splits in {fill, min(fill, 8)}:                        # the norm adds planes eight at a time
            per_slice = -(-k_blocks // splits)
            planes = -(-k_blocks // per_slice)
            rounds = -(-tiles * planes // SM_COUNT)
            cost = (rounds * per_slice * per_block + planes * (2.0 * M * N * 4 / 3.5e6)
                    + 2.0 * (-(-planes // 8) - 1))
            if planes > 1 and (best is None or cost < best[0]):
                best = (cost, tile, splits)
    if best is None or best[0] >= whole:
        return 0, 1                                               # not worth cutting
    return best[1], best[2]


def gemm_bf16_slices(x: torch.Tensor, weight: torch.Tensor) -> Optional[torch.Tensor]:
    """x . weight^T as float32 partial products over K slices, [slices, M, N], whose sum in plane
    order is the product; None when this shape is not worth cutting (the caller then adds the
    whole product in place). For products that go into the residual stream."""
    M, K = x.shape
    N = weight.shape[0]
    lib = library.load()
    stream_ok, umma_ok = _fast_kernels(x, weight, lib)
    if not stream_ok:
        if not umma_ok or M <= 64:
            return None
        # A short prompt (a few hundred rows): few tiles and a long K leave most SMs idle (the 2048 x
        # 8192 product of a 128-token prompt: 16 CTAs, 42 us), so K is cut until the items fill the
        # SMs once, no slice shorter than 256 (the same product in 9 slices: 12 us).
        tile, splits = _sliced_plan(M, N, K)
        planes = lib.lrm_gemm_bf16_umma_slices(K, splits) if splits > 1 else 1
        if planes <= 1:
            return None
        out = torch.empty((planes, M, N), dtype=torch.float32, device=x.device)
        mark_status_dirty()
        _done(lib.lrm_gemm_bf16_umma_rows(_ptr(x), _ptr(weight), _ptr(out), M, M, N, K, 4, tile, splits,
                                          _ptr(_status_word(x.device)), _stream()), "gemm_bf16_umma")
        return out
    use_umma, splits = False, 1
    if umma_ok and M > STREAM_ROWS and not force_stream:
        use_umma, splits = _few_rows_plan(M, N, K, 4)
    if use_umma:
        planes = lib.lrm_gemm_bf16_umma_slices(K, splits)
        if planes <= 1:
            return None
        out = torch.empty((planes, M, N), dtype=torch.float32, device=x.device)
        mark_status_dirty()
        held = (x.untyped_storage().nbytes() // x.element_size() - x.storage_offset()) // K
        _done(lib.lrm_gemm_bf16_umma_rows(_ptr(x), _ptr(weight), _ptr(out), M, min(max(M, 32), max(M, held)), N, K,
                                          4, 0 if umma_width is None else tile_choice(M, N, K, 4), splits,
                                          _ptr(_status_word(x.device)), _stream()), "gemm_bf16_umma")
        return out
    warps, wanted = stream_shape if stream_shape is not None else (0, 0)
    planes = lib.lrm_gemm_bf16_stream_slices(M, N, K, wanted)
    if planes <= 1:
        return None
    out = torch.empty((planes, M, N), dtype=torch.float32, device=x.device)
    _done(lib.lrm_gemm_bf16_stream_shaped(_ptr(x), _ptr(weight), _ptr(out), M, N, K, 4, warps, wanted, _stream()),
          "gemm_bf16_stream")
    return out


def gemm_bf16_qkv(x: torch.Tensor, weight: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                  kv, dest_rows: Optional[torch.Tensor], table: Optional[torch.Tensor]) -> bool:
    """A prompt's fused q|k|v projection with rotation and stores in the product's epilogue:
    q [T, Hq, d], k, v [T, Hk, d] packed, and k, v into the paged cache view `kv` at `dest_rows`
    (both None: no cache). `table`: float32 [T, d/2, 2] (cos, sin), or None for no rotation.
    False (nothing launched) where only the separate kernels take the shape."""
    M, K = x.shape
    N = weight.shape[0]
    T, Hq, d = q.shape
    Hk = k.shape[1]
    lib = library.load()
    _, umma_ok = _fast_kernels(x, weight, lib)
    if not umma_ok or no_fused_rope or M <= 64 or d not in (64, 128) or N != (Hq + 2 * Hk) * d:
        return False
    tile = tile_choice(M, N, K, 0, pair_room(), multiple_of=d)
    pages = (_ptr(kv.k), _ptr(kv.v), _ptr(dest_rows), kv.page_size) if kv is not None else (None, None, None, 1)
    mark_status_dirty()
    if tile == PAIR:
        _done(lib.lrm_gemm_bf16_umma_pair_qkv(_ptr(x), _ptr(weight), M, N, K, _ptr(q), _ptr(k), _ptr(v), pages[0],
                                              pages[1], pages[2], _ptr(table), Hq, Hk, d, pages[3],
                                              _ptr(_status_word(x.device)), _stream()), "gemm_bf16_umma_pair_qkv")
    else:
        _done(lib.lrm_gemm_bf16_umma_qkv(_ptr(x), _ptr(weight), M, N, K, tile, _ptr(q), _ptr(k), _ptr(v), pages[0],
                                         pages[1], pages[2], _ptr(table), Hq, Hk, d, pages[3],
                                         _ptr(_status_word(x.device)), _stream()), "gemm_bf16_umma_qkv")
    return True


no_fused_rope = False  # tests: keep rotation and stores in their own launch


def gemm_bf16(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, mode: int) -> None:
    """out (mode 0 bf16 store, 1 f32 store, 2 f32 add in place, 3 silu gate) = x . weight^T."""
    M, K = x.shape
    N = weight.shape[0]
    lib = library.load()
    stream_ok, umma_ok = _fast_kernels(x, weight, lib)
    tile, splits = tile_choice(M, N, K, mode, pair_room() if umma_ok and M > 64 else 0), 1
    if stream_ok and umma_ok and M > STREAM_ROWS and not force_stream:
        use_umma, splits = _few_rows_plan(M, N, K, mode)
        stream_ok = not use_umma
        tile = 0 if umma_width is None else tile
    if stream_ok:
        warps = stream_shape[0] if stream_shape is not None else 0
        _done(lib.lrm_gemm_bf16_stream_shaped(_ptr(x), _ptr(weight), _ptr(out), M, N, K, mode, warps, 0,
                                              _stream()), "gemm_bf16_stream")
        return
    if umma_ok and tile == PAIR:
        mark_status_dirty()
        _done(lib.lrm_gemm_bf16_umma_pair(_ptr(x), _ptr(weight), _ptr(out), M, N, K, mode,
                                          _ptr(_status_word(x.device)), _stream()), "gemm_bf16_umma_pair")
        return
    if umma_ok:
        mark_status_dirty()
        # rows of x that its storage holds beyond M may be named in the tensor map (see the kernel)
        held = (x.untyped_storage().nbytes() // x.element_size() - x.storage_offset()) // K
        _done(lib.lrm_gemm_bf16_umma_rows(_ptr(x), _ptr(weight), _ptr(out), M, min(max(M, 32), max(M, held)), N, K,
                                          mode, tile, splits, _ptr(_status_word(x.device)), _stream()),
              "gemm_bf16_umma")
        return
    _done(lib.lrm_gemm_bf16_mma(_ptr(x), _ptr(weight), _ptr(out), M, N, K, mode, _stream()),
          "gemm_bf16_mma")
