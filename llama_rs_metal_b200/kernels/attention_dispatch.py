"""Which attention kernel runs for a geometry.

The row-wise kernel (csrc/attention_rowwise.cu) takes every head size up to
512 and both dtypes, and is the only attention of the float32 path. bfloat16
prompts with head size 64 or 128 run the TMA + tcgen05 kernel
(csrc/attention_prefill_umma.cu); bfloat16 with head size 32, 64 or 128 and
64-token pages otherwise runs the warp-level tiled kernels (csrc/attention_tiled.cu).
A bfloat16 decode step of a layer that writes its own unwindowed cache runs rotation,
cache write, attention and the merge of the splits as one cluster kernel
(csrc/attention_decode_cluster.cu). A step that appends several tokens to started
sequences stores its keys first and attends over the cache (row-wise, or the tiled
extend kernel in bfloat16).

`attend` is the one call a mixer makes: it takes the step's projection and picks
rotation, cache write and attention kernels for the step's phase and geometry.
"""
from __future__ import annotations

import ctypes
import os

import torch

from . import library
from .ops import _code, _done, _ptr, _stream  # noqa: PLC2701

SM_COUNT = 148
force_rowwise = False  # tests switch the tiled kernels off to compare both paths
force_warp_level = False  # tests keep prompts off the tcgen05 kernel to cover the warp-level one
force_unfused_decode = False  # tests keep decode steps on the separate rotation / attention / merge kernels
force_cluster_size = None  # tests fix the CTAs per cluster of the fused decode kernel
prefill_kernel = None  # tests pin the tcgen05 prompt kernel: "pingpong" or "single" (None: the rule in prefill())


def _tiled(q, page_size: int) -> bool:
    return (not force_rowwise and q.dtype == torch.bfloat16
            and bool(library.load().lrm_attention_tiled_supports(q.shape[2], page_size)))


def prefill(q, k, v, out, cu_seqlens, seq_of_token, max_seq_len: int, scale: float, window: int) -> None:
    T, Hq, d = q.shape
    lib = library.load()
    aligned = all(t.data_ptr() % 16 == 0 for t in (q, k, v, out))
    if (not force_rowwise and not force_warp_level and q.dtype == torch.bfloat16 and aligned
            and lib.lrm_attention_prefill_umma_supports(d)):
        from . import gemm_dispatch
        gemm_dispatch.mark_status_dirty()
        # Two tcgen05 kernels. The one that keeps probabilities and output in tensor memory wins on
        # long prompts and on batches of prompts: at head size 128 (one query tile per CTA on key tiles
        # of 64 up to 2,304 tokens, two query tiles taking turns beyond) from 1,536 tokens on (2,048
        # tokens 60 against 86 us, 953 against 582 TFLOP/s at 32,768); at head size 64 (four CTAs per SM on key tiles of 64) beyond 2,048 tokens (3,072
        # tokens 78 against 100 us, 681 against 534 TFLOP/s at 32,768) and whenever several prompts
        # are packed (four of 512 tokens 20 against 29 us, eight of 128 tokens 9.5 against 11.1). A
        # single short prompt is bound by the chain of key tiles of its last query tile, which the
        # older kernel, with two threads per row, walks a little faster (1,024 tokens 24 against 26 us).
        # Packed prompts go to the newer kernel at head size 128 too (four of 512 tokens 33 against 46 us).
        # (several prompts: the packed tokens are well more than the longest prompt; a short prompt
        # filled up to whole rows with a few tokens of padding does not count)
        pingpong = (max_seq_len >= 1536 if d == 128 else max_seq_len > 2048) or 4 * T >= 5 * max_seq_len
        if prefill_kernel is not None:
            pingpong = prefill_kernel == "pingpong"
        if pingpong:
            _done(lib.lrm_attention_prefill_pingpong(_ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(cu_seqlens), T,
                                                     cu_seqlens.numel() - 1, max_seq_len, Hq, k.shape[1], d,
                                                     ctypes.c_float(scale), window,
                                                     _ptr(gemm_dispatch._status_word(q.device)), _stream()),
                  "attention_prefill_pingpong")
            return
        _done(lib.lrm_attention_prefill_umma(_ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(cu_seqlens), T,
                                             cu_seqlens.numel() - 1, max_seq_len, Hq, k.shape[1], d,
                                             ctypes.c_float(scale), window,
                                             _ptr(gemm_dispatch._status_word(q.device)), _stream()),
              "attention_prefill_umma")
        return
    if _tiled(q, 64):
        _done(lib.lrm_attention_prefill_tiled(_ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(cu_seqlens),
                                              cu_seqlens.numel() - 1, max_seq_len, Hq, k.shape[1], d,
                                              ctypes.c_float(scale), window, _stream()),
              "attention_prefill_tiled")
        return
    _done(lib.lrm_attention_packed_rowwise(_ptr(q), _ptr(k), _ptr(v), _ptr(out), _code(q.dtype),
                                           _ptr(cu_seqlens), _ptr(seq_of_token), T, Hq, k.shape[1], d,
                                           ctypes.c_float(scale), window, _stream()),
          "attention_packed_rowwise")


CTAS_PER_SM = 4  # decode attention CTAs wanted per SM (each keeps one 64-key K/V tile in flight)


def decode_splits(seqs: int, kv_heads: int, group: int, max_kv_len: int, window: int) -> int:
    """Splits of the key range so that about CTAS_PER_SM CTAs per SM stream the cache."""
    ctas = seqs * kv_heads * -(-group // 16)
    keys = min(max_kv_len, window + 63) if window > 0 else max_kv_len
    pages = max(1, -(-keys // 64))
    return max(1, min(pages, -(-CTAS_PER_SM * SM_COUNT // ctas)))


def decode(q, kv, out, slots, kv_lens, max_kv_len: int, scale: float, window: int) -> None:
    B, Hq, d = q.shape
    lib = library.load()
    if _tiled(q, kv.page_size):
        splits = decode_splits(B, kv.kv_heads, Hq // kv.kv_heads, max_kv_len, window)
        partials = torch.empty((B, Hq, splits, d + 2), dtype=torch.float32, device=q.device)
        _done(lib.lrm_attention_decode_tiled(_ptr(q), _ptr(kv.k), _ptr(kv.v), _ptr(partials), _ptr(out),
                                             _ptr(kv.page_table), kv.page_table.shape[1], _ptr(slots),
                                             _ptr(kv_lens), B, Hq, kv.kv_heads, d, kv.page_size,
                                             ctypes.c_float(scale), window, splits, _stream()),
              "attention_decode_tiled", launches=2)
        return
    _done(lib.lrm_attention_paged_rowwise(_ptr(q), _ptr(kv.k), _ptr(kv.v), _ptr(out), _code(q.dtype),
                                          _ptr(kv.page_table), kv.page_table.shape[1], _ptr(slots),
                                          _ptr(kv_lens), None, None, B, Hq, kv.kv_heads, d, kv.page_size,
                                          ctypes.c_float(scale), window, _stream()),
          "attention_paged_rowwise")


def extend(q, kv, out, cu_seqlens, seq_of_token, positions, slots, kv_lens, max_seq_len: int, scale: float,
           window: int) -> None:
    """Packed queries, several per sequence, over the cache that already holds the step's keys."""
    T, Hq, d = q.shape
    lib = library.load()
    if _tiled(q, kv.page_size):
        _done(lib.lrm_attention_extend_tiled(_ptr(q), _ptr(kv.k), _ptr(kv.v), _ptr(out), _ptr(cu_seqlens),
                                             _ptr(kv.page_table), kv.page_table.shape[1], _ptr(slots),
                                             _ptr(kv_lens), cu_seqlens.numel() - 1, max_seq_len, Hq,
                                             kv.kv_heads, d, kv.page_size, ctypes.c_float(scale), window,
                                             _stream()), "attention_extend_tiled")
        return
    # the same arithmetic, key by key in ascending order, as the packed row-wise kernel: in
    # float32 a prompt cut into portions gives the bits of the whole prompt
    _done(lib.lrm_attention_paged_rowwise(_ptr(q), _ptr(kv.k), _ptr(kv.v), _ptr(out), _code(q.dtype),
                                          _ptr(kv.page_table), kv.page_table.shape[1], _ptr(slots),
                                          _ptr(kv_lens), _ptr(seq_of_token), _ptr(positions), T, Hq,
                                          kv.kv_heads, d, kv.page_size, ctypes.c_float(scale), window,
                                          _stream()), "attention_paged_rowwise")


_cluster_room = {}


def _resident_clusters(head_dim: int, cluster: int, rows: int) -> int:
    """Clusters of this size, with `rows` query heads per kv head in a CTA, that the device holds
    at once (the region that partials are sent into grows with both); 0: cannot be launched."""
    key = (head_dim, cluster, rows)
    if key not in _cluster_room:
        _cluster_room[key] = int(library.load().lrm_attention_decode_cluster_resident(head_dim, cluster, rows))
    return _cluster_room[key]


def decode_fused_supported(dtype, head_dim: int, page_size: int, rotary: int, window) -> bool:
    """True when one cluster kernel can do rotation, cache write, attention and merge."""
    return (not force_rowwise and not force_unfused_decode and dtype == torch.bfloat16 and not window
            and bool(library.load().lrm_attention_decode_cluster_supports(head_dim, page_size, rotary)))


def decode_prefers_fused(seqs: int, kv_heads: int, group: int, head_dim: int, max_kv_len: int,
                         fill: int = 4) -> bool:
    """Whether the one-launch cluster kernel or the separate kernels are the faster way through a
    decode step's attention. A cluster has at most 16 CTAs, and a CTA keeps two pages in flight,
    which is worth 16-20 GB/s at head size 64 (25-30 at 128): a few sequences with a long context leave the
    cluster kernel with too few CTAs to draw the memory's bandwidth (measured: 112 CTAs 2.1 TB/s,
    224 CTAs 3.5, 320 CTAs 5.1, from 384 CTAs on 6.0-6.2), while the separate kernels cut a sequence
    into as many splits as fill the device and read at 6.6 TB/s (6.0 at head size 128), unless there are so many
    (sequence, head) pairs that each gets only two or three splits (256 pairs and more: 4.7-5.6).
    Against that stand their three launches: about 17 us before anything else counts, 8 us for the
    cluster kernel plus 0.35 us per page a CTA walks. Whole decode steps of the 1B shape, cluster
    kernel against separate kernels, ms: batch 1 at 16,000 keys 0.94 / 0.99, at 64,000 1.72 / 1.24;
    batch 4: 1.19 / 1.15 and 2.43 / 2.06; batch 8: 1.46 / 1.43 and 3.69 / 3.34; batch 32 at 16,000:
    3.85 / 4.50; batch 64: 6.92 / 7.29; at 4,000 keys the cluster kernel wins at every batch."""
    if force_cluster_size is not None:
        return True
    pages = max(1, -(-max_kv_len // 64))
    cluster = decode_cluster_size(seqs, kv_heads, group, head_dim, max_kv_len, fill)
    pairs = seqs * kv_heads * -(-group // 16)
    page_bytes = 4.0 * 64 * head_dim                       # a page of keys and one of values
    data = pairs * pages * page_bytes                      # bytes; rates below in bytes per us
    per_cta = 16e3 + 70.0 * head_dim                       # 20 GB/s at head size 64, 25 at 128
    fused = max(8.0 + 0.35 * -(-pages // cluster), data / min(6.1e6, pairs * cluster * per_cta))
    separate = max(17.0, data / (5.0e6 if pairs > 128 else 6.6e6 if head_dim <= 64 else 6.0e6) + 3.0)
    return fused <= separate


MAX_CLUSTER = 14  # clusters of 15 and 16 CTAs were measured slower as soon as a few hundred CTAs run


def decode_cluster_size(seqs: int, kv_heads: int, group: int, head_dim: int, max_kv_len: int, fill: int = 4) -> int:
    """CTAs per (sequence, kv head): any size up to MAX_CLUSTER (not only powers of two). Measured
    over batches of 1-32 and 600-8,000 keys, the kernel is fastest with about 400 CTAs in all at
    head size 64 (under 3 per SM, of the 4 that fit), about 500 when each walks many pages; more
    than fit at once cost a second round. `fill`: the sequences' mean length in quarters of the
    longest (4: about equal). Unequal sequences are handed out longest first, so the clusters that
    wait for room are those of the short sequences, and a size more pays: 16 sequences of 64-4,096
    keys, 1B shape: 1.20 ms per step with clusters of 4 against 1.25 with 3; 3B shape: 3.05-3.06 with
    5 or 4 against 3.16 with 3 (and 1.24-1.27 / 3.18 without the ordering, whatever the size)."""
    if force_cluster_size is not None:
        return force_cluster_size
    clusters = seqs * kv_heads * -(-group // 16)
    pages = max(1, -(-max_kv_len // 64))
    slots = (CTAS_PER_SM if head_dim <= 64 else 3) * SM_COUNT
    size = max(1, min(int(0.68 * slots / clusters + 0.5), pages, MAX_CLUSTER))
    if pages >= 16 * size:  # long rows of pages per CTA: bandwidth counts more than balance
        size = max(1, min(int(0.85 * slots / clusters + 0.5), pages, MAX_CLUSTER))
    while size > 1 and clusters > _resident_clusters(head_dim, size, min(group, 16)):
        size -= 1
    if fill < 4 and seqs > 1 and size < min(pages, MAX_CLUSTER):
        # as many more clusters may wait their turn as the short sequences leave room for
        if clusters * fill <= 4 * _resident_clusters(head_dim, size + 1, min(group, 16)):
            size += 1
    return size


def decode_fused(qkv, positions, inv_freq, rotary: int, kv, dest_rows, out, slots, kv_lens, max_kv_len: int,
                 q_heads: int, scale: float, order=None, fill: int = 4) -> None:
    B = qkv.shape[0]
    d = kv.head_dim
    cluster = decode_cluster_size(B, kv.kv_heads, q_heads // kv.kv_heads, d, max_kv_len, fill if order is not None else 4)
    _done(library.load().lrm_attention_decode_cluster(
        _ptr(qkv), _ptr(positions), _ptr(inv_freq), rotary, _ptr(kv.k), _ptr(kv.v), _ptr(dest_rows), _ptr(out),
        _ptr(kv.page_table), kv.page_table.shape[1], _ptr(slots), _ptr(kv_lens), B, q_heads, kv.kv_heads, d,
        kv.page_size, ctypes.c_float(scale), cluster, _ptr(order), _stream()), "attention_decode_cluster")


# --------------------------------------------------------------------------- one call for a mixer
def attend(projected, *, q_heads: int, kv_heads: int, head_dim: int, rotary, ctx, cache, writes_cache: bool,
           cache_entry: int, scale: float, window, projection=None):
    """A layer's attention for one step: position rotation, cache write and attention, with the
    kernels chosen here for the step's phase, dtype and geometry. -> mixed heads [T, q_heads * d].

    projected: the step's fused [T, (q_heads + 2 kv_heads) * d] q|k|v projection when the layer
        writes its cache entry, else its [T, q_heads * d] queries (the entry was filled, in this
        step, by the layer that owns it).
    rotary: (inverse frequencies float32 [R/2], R) for a split-half rotation applied here, or None
        (no rotation: another scheme already transformed q and k, or there is none).
    ctx: the StepContext; cache: the KeyValueView of `cache_entry`; window: keys a query sees, or None.
    projection: (x, weight) instead of `projected` (then None) when nothing stands between the
        projection and the rotation: a prompt's product then rotates and stores in its epilogue.
    """
    from . import ops
    inv_freq, width = rotary if rotary is not None else (None, 0)
    phase = ctx.phase
    if projection is not None:
        x, weight = projection
        if (phase == "prefill" and writes_cache and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
                and width in (0, head_dim)):
            table = None
            if inv_freq is not None:   # one table of cosines and sines per step and rotation
                table = ctx.scratch.get(("rope_table", id(inv_freq)))
                if table is None:
                    table = ctx.scratch[("rope_table", id(inv_freq))] = ops.rope_table(ctx.positions, inv_freq)
            fused = ops.linear_rope_store(x, weight, q_heads, kv_heads, head_dim, table, cache,
                                          ctx.dest_rows[cache.group] if cache is not None else None)
            if fused is not None:
                q, k, v = fused
                ctx.fresh_kv[cache_entry] = (k, v)
                return ops.attention_prefill(q, k, v, ctx.cu_seqlens, ctx.seq_of_token, ctx.max_seq_len, scale, window)
        projected = ops.linear(x, weight)
    if writes_cache:
        if (phase == "decode" and cache is not None and projected.dtype == torch.bfloat16
                and decode_fused_supported(projected.dtype, head_dim, cache.page_size, width,
                                           window or cache.window)
                and decode_prefers_fused(projected.shape[0], kv_heads, q_heads // kv_heads, head_dim,
                                         ctx.max_kv_len, ctx.kv_fill)):
            # rotation, cache write, attention and the merge of the splits in one launch
            # the order comes with the step's arrays: the kernel reads it before it waits
            order = ctx.longest_first if projected.shape[0] > 1 else None
            return ops.attention_decode_fused(projected, q_heads, inv_freq, width, ctx.positions, cache,
                                              ctx.dest_rows[cache.group], ctx.slots, ctx.kv_lens,
                                              ctx.max_kv_len, scale, order, ctx.kv_fill)
        prefill = phase == "prefill"
        q, k, v = ops.rope_store(projected, q_heads, kv_heads, head_dim, inv_freq, width, ctx.positions,
                                 kv=cache, dest_rows=ctx.dest_rows[cache.group] if cache is not None else None,
                                 keep_packed=prefill)
        if prefill:
            ctx.fresh_kv[cache_entry] = (k, v)
    else:
        q, _, _ = ops.rope_store(projected, q_heads, 0, head_dim, inv_freq, width, ctx.positions,
                                 keep_packed=False)
        if phase == "prefill":
            k, v = ctx.fresh_kv[cache_entry]
    if phase == "prefill":
        return ops.attention_prefill(q, k, v, ctx.cu_seqlens, ctx.seq_of_token, ctx.max_seq_len, scale, window)
    if phase == "decode":
        return ops.attention_decode(q, cache, ctx.slots, ctx.kv_lens, ctx.max_kv_len, scale, window)
    return ops.attention_extend(q, cache, ctx.cu_seqlens, ctx.seq_of_token, ctx.positions, ctx.slots,
                                ctx.kv_lens, ctx.max_seq_len, scale, window)
