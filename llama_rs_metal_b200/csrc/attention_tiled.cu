// Tiled bfloat16 attention on the warp-level tensor path (mma.sync m16n8k16,
// ldmatrix, cp.async), float32 softmax and accumulation.
//
//  * prefill: causal grouped-query flash attention over a step's own packed
//    q, k, v (ragged batch, every sequence starts at position 0). One CTA = 64
//    queries of one head; K/V arrive in 64-key tiles, double buffered.
//  * extend: the same flash attention for a portion of several tokens appended to started
//    sequences: queries are the step's packed tokens, keys and values come from the paged
//    cache (which already holds the portion's own), one 64-key page per tile.
//  * decode: one query per sequence over the paged cache, split over the keys.
//    One CTA = (sequence, kv head, split); its 4 warps each take 16 keys of
//    every 64-key page, so K/V are read once for all query heads of the group.
//    The warps' unnormalised partials (acc, max, mass) are combined in shared memory,
//    the CTA leaves one partial per split, and a second kernel merges the splits in
//    order: out = sum acc_i 2^(m_i-M) / sum l_i 2^(m_i-M).
//    (Merging in the last CTA to arrive, found with a global counter, was tried and
//    was slower than the separate launch: its serial tail costs more than a launch.)
//    (reference: crates/metal-backend/src/shaders/attention.metal:61-121 splits
//    the context the same way, one SIMD group per chunk.)
//
// Scores are kept in the log2 domain: s2 = (q.k) * scale * log2(e), p = 2^(s2 - m2).
// Rows of a tile beyond a sequence's length are zero-filled on the way into
// shared memory, so stale cache contents (even NaN bit patterns) never reach a
// product. Head sizes 32, 64 and 128; other sizes use the row-wise kernel.
#include "attention_mma.cuh"

namespace {

// --------------------------------------------------------------------------- prefill
template <int D>
__global__ __launch_bounds__(kThreads) void attention_prefill_tiled_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
    const __nv_bfloat16* __restrict__ v, __nv_bfloat16* __restrict__ out,
    const int* __restrict__ cu_seqlens, int q_heads, int kv_heads, float scale_log2, int window) {
  constexpr int STRIDE = D + 8, TILE = kTile * STRIDE;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // [2][64][STRIDE]
  __nv_bfloat16* Vs = Ks + 2 * TILE;

  pdl_wait();
  // CTAs are handed out in the order x, y, z: the last query tile (the longest row of work under
  // the causal mask) of every head and sequence first, so the grid's tail is made of short CTAs.
  const int qt = gridDim.z - 1 - blockIdx.z;
  const int h = blockIdx.x, b = blockIdx.y;
  const int start = cu_seqlens[b], len = cu_seqlens[b + 1] - start;
  const int q0 = qt * kTile;
  if (q0 >= len) return;
  const int kh = h / (q_heads / kv_heads);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int row0 = q0 + 16 * warp;  // this warp's first query (position in the sequence)

  uint32_t qa[D / 16][4];
  load_q<D>(qa, q + (static_cast<size_t>(start + row0) * q_heads + h) * D,
            static_cast<size_t>(q_heads) * D, len - row0);
  float o[D / 8][4];
#pragma unroll
  for (int dn = 0; dn < D / 8; ++dn)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[dn][e] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  const int kt_first = window > 0 ? max(0, q0 - window + 1) / kTile : 0;
  const int kt_last = qt;
  const size_t kv_pitch = static_cast<size_t>(kv_heads) * D;
  auto issue = [&](int kt, int stage) {
    const size_t base = (static_cast<size_t>(start + kt * kTile) * kv_heads + kh) * D;
    load_tile<D>(Ks + stage * TILE, k + base, kv_pitch, len - kt * kTile);
    load_tile<D>(Vs + stage * TILE, v + base, kv_pitch, len - kt * kTile);
    cp_async_commit();
  };
  issue(kt_first, 0);
  for (int kt = kt_first; kt <= kt_last; ++kt) {
    const int stage = (kt - kt_first) & 1;
    if (kt < kt_last) {
      issue(kt + 1, stage ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    float s[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
    scores<D, 8>(s, qa, Ks + stage * TILE);
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = kt * kTile + 8 * nt + 2 * t + (e & 1);
        const int query = row0 + g + 8 * (e >> 1);
        const bool visible = key <= query && (window <= 0 || key > query - window);
        s[nt][e] = visible ? s[nt][e] * scale_log2 : -INFINITY;
      }
    }
    softmax_update<D, 8>(s, o, m, l);
    weighted_values<D, 8>(o, s, Vs + stage * TILE);
    __syncthreads();
  }
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    float total = l[half];
    total += __shfl_xor_sync(0xffffffffu, total, 1);
    total += __shfl_xor_sync(0xffffffffu, total, 2);
    const int row = row0 + g + 8 * half;
    if (row >= len) continue;
    const float inv = 1.0f / total;
    __nv_bfloat16* dst = out + (static_cast<size_t>(start + row) * q_heads + h) * D;
#pragma unroll
    for (int dn = 0; dn < D / 8; ++dn)
      *reinterpret_cast<uint32_t*>(dst + 8 * dn + 2 * t) =
          pack_bf16(o[dn][2 * half] * inv, o[dn][2 * half + 1] * inv);
  }
}

// --------------------------------------------------------------------------- extend
// Queries: the step's packed tokens (sequence b brings n = cu_seqlens[b+1] - cu_seqlens[b] of
// them, standing at positions kv_lens[b] - n .. kv_lens[b] - 1). Keys and values: the paged cache,
// which holds every position up to kv_lens[b] - 1, this step's included. One CTA = 64 queries of one
// head; a key tile is one page.
template <int D>
__global__ __launch_bounds__(kThreads) void attention_extend_tiled_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pages,
    const __nv_bfloat16* __restrict__ v_pages, __nv_bfloat16* __restrict__ out,
    const int* __restrict__ cu_seqlens, const int* __restrict__ page_table, int table_stride,
    const int* __restrict__ slots, const int* __restrict__ kv_lens, int q_heads, int kv_heads,
    float scale_log2, int window) {
  constexpr int STRIDE = D + 8, TILE = kTile * STRIDE;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // [2][64][STRIDE]
  __nv_bfloat16* Vs = Ks + 2 * TILE;

  pdl_wait();
  const int qt = gridDim.z - 1 - blockIdx.z;  // longest rows of work first
  const int h = blockIdx.x, b = blockIdx.y;
  const int start = cu_seqlens[b], n = cu_seqlens[b + 1] - start;
  const int q0 = qt * kTile;
  if (q0 >= n) return;
  const int len = kv_lens[b], before = len - n;
  const int kh = h / (q_heads / kv_heads);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int row0 = q0 + 16 * warp;  // this warp's first query, counted within the portion
  const int* table = page_table + static_cast<size_t>(slots[b]) * table_stride;

  uint32_t qa[D / 16][4];
  load_q<D>(qa, q + (static_cast<size_t>(start + row0) * q_heads + h) * D,
            static_cast<size_t>(q_heads) * D, n - row0);
  float o[D / 8][4];
#pragma unroll
  for (int dn = 0; dn < D / 8; ++dn)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[dn][e] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  // keys the tile's queries see: from the first query's window to the last query's own position
  const int first_key = window > 0 ? max(0, before + q0 - window + 1) : 0;
  const int kt_first = first_key / kTile;
  const int kt_last = (before + min(q0 + kTile, n) - 1) / kTile;
  auto issue = [&](int kt, int stage) {
    const int page = table[kt];
    const size_t base = (static_cast<size_t>(max(page, 0)) * kv_heads + kh) * kTile * D;
    // rows behind the sequence's end, before the window, or of a page the sequence does not hold
    // are zero-filled (the mask hides them; stale bits must not reach a product)
    const int valid = page >= 0 ? len - kt * kTile : 0;
    load_page<D>(Ks + stage * TILE, k_pages + base, valid, first_key - kt * kTile);
    load_page<D>(Vs + stage * TILE, v_pages + base, valid, first_key - kt * kTile);
    cp_async_commit();
  };
  issue(kt_first, 0);
  for (int kt = kt_first; kt <= kt_last; ++kt) {
    const int stage = (kt - kt_first) & 1;
    if (kt < kt_last) {
      issue(kt + 1, stage ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    float s[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
    scores<D, 8>(s, qa, Ks + stage * TILE);
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = kt * kTile + 8 * nt + 2 * t + (e & 1);
        const int query = before + row0 + g + 8 * (e >> 1);  // position in the sequence
        const bool visible = key <= query && (window <= 0 || key > query - window);
        s[nt][e] = visible ? s[nt][e] * scale_log2 : -INFINITY;
      }
    }
    softmax_update<D, 8>(s, o, m, l);
    weighted_values<D, 8>(o, s, Vs + stage * TILE);
    __syncthreads();
  }
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    float total = l[half];
    total += __shfl_xor_sync(0xffffffffu, total, 1);
    total += __shfl_xor_sync(0xffffffffu, total, 2);
    const int row = row0 + g + 8 * half;
    if (row >= n) continue;
    const float inv = 1.0f / total;
    __nv_bfloat16* dst = out + (static_cast<size_t>(start + row) * q_heads + h) * D;
#pragma unroll
    for (int dn = 0; dn < D / 8; ++dn)
      *reinterpret_cast<uint32_t*>(dst + 8 * dn + 2 * t) =
          pack_bf16(o[dn][2 * half] * inv, o[dn][2 * half + 1] * inv);
  }
}

// --------------------------------------------------------------------------- decode
// partial layout: [sequence][q head][split][D + 2] float32,
// element D = running max (log2 domain), element D + 1 = mass.
template <int D>
__global__ __launch_bounds__(kThreads) void attention_decode_tiled_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pages,
    const __nv_bfloat16* __restrict__ v_pages, float* __restrict__ partials,
    const int* __restrict__ page_table, int table_stride, const int* __restrict__ slots,
    const int* __restrict__ kv_lens, int q_heads, int kv_heads, int row_groups, float scale_log2,
    int window, int n_splits) {
  // no early griddepcontrol.launch_dependents: the kernels after attention trigger at once in their
  // turn, and a whole layer's kernels scheduled behind a running attention made decode steps slower
  constexpr int STRIDE = D + 8, TILE = kTile * STRIDE;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* Vs = Ks + 2 * TILE;
  const int rg = blockIdx.x % row_groups;
  const int kh = (blockIdx.x / row_groups) % kv_heads;
  const int b = blockIdx.x / (row_groups * kv_heads);
  const int split = blockIdx.y;
  const int group = q_heads / kv_heads;
  const int head0 = kh * group + 16 * rg;          // first query head of this CTA
  const int rows = min(16, group - 16 * rg);       // query heads it owns
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;

  const int len = kv_lens[b];
  const int first_key = window > 0 ? max(0, len - window) : 0;
  const int page_first = first_key / kTile, page_end = (len + kTile - 1) / kTile;
  const int n_pages = page_end - page_first;
  const int per_split = (n_pages + n_splits - 1) / n_splits;
  const int p_begin = page_first + split * per_split;
  const int p_end = min(page_end, p_begin + per_split);
  const int* table = page_table + static_cast<size_t>(slots[b]) * table_stride;

  auto issue = [&](int page_index, int stage) {
    const size_t page = static_cast<size_t>(table[page_index]);
    const size_t base = (page * kv_heads + kh) * kTile * D;
    load_page<D>(Ks + stage * TILE, k_pages + base, len - page_index * kTile, first_key - page_index * kTile);
    load_page<D>(Vs + stage * TILE, v_pages + base, len - page_index * kTile, first_key - page_index * kTile);
    cp_async_commit();
  };
  // Lengths, slots and the page table were set before the step; only q and the newest
  // key/value row (in the sequence's last page) come from the kernel before this one. A first
  // page that is not the last one can therefore be fetched before waiting for that kernel.
  const bool early = p_begin < p_end && p_begin != page_end - 1;
  if (early) issue(p_begin, 0);
  pdl_wait();
  if (!early && p_begin < p_end) issue(p_begin, 0);

  uint32_t qa[D / 16][4];
  load_q<D>(qa, q + (static_cast<size_t>(b) * q_heads + head0) * D, D, rows);
  float o[D / 8][4];
#pragma unroll
  for (int dn = 0; dn < D / 8; ++dn)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[dn][e] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  for (int p = p_begin; p < p_end; ++p) {
    const int stage = (p - p_begin) & 1;
    cp_async_wait<0>();  // page p is here
    __syncthreads();     // ... for every thread, and everyone is done with page p - 1
    if (p + 1 < p_end) issue(p + 1, stage ^ 1);  // into the buffer page p - 1 was in
    float s[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
    scores<D, 2>(s, qa, Ks + stage * TILE + 16 * warp * STRIDE);
    if ((p + 1) * kTile <= len && p * kTile >= first_key) {  // a page wholly inside the visible range
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[nt][e] *= scale_log2;
    } else {
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = p * kTile + 16 * warp + 8 * nt + 2 * t + (e & 1);
          const bool visible = key < len && key >= first_key;
          s[nt][e] = visible ? s[nt][e] * scale_log2 : -INFINITY;
        }
      }
    }
    if (rows > 8) softmax_update<D, 2, 2>(s, o, m, l);
    else softmax_update<D, 2, 1>(s, o, m, l);  // query heads 8..15 of the tile are padding
    weighted_values<D, 2>(o, s, Vs + stage * TILE + 16 * warp * STRIDE);
  }

  // Combine the four warps (each saw 16 keys of every page) through shared memory, which the
  // K/V tiles no longer need: per warp [16 rows][D + 2] floats.
  __syncthreads();
  float* stage = reinterpret_cast<float*>(smem_raw) + warp * 16 * (D + 2);
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    float total = l[half];
    total += __shfl_xor_sync(0xffffffffu, total, 1);
    total += __shfl_xor_sync(0xffffffffu, total, 2);
    float* dst = stage + (g + 8 * half) * (D + 2);
#pragma unroll
    for (int dn = 0; dn < D / 8; ++dn)
      *reinterpret_cast<float2*>(dst + 8 * dn + 2 * t) = make_float2(o[dn][2 * half], o[dn][2 * half + 1]);
    if (t == 0) {
      dst[D] = m[half];
      dst[D + 1] = total;
    }
  }
  __syncthreads();
  const float* all = reinterpret_cast<const float*>(smem_raw);
  for (int item = threadIdx.x; item < rows * (D + 2); item += kThreads) {
    const int r = item / (D + 2), c = item % (D + 2);
    float mw[4], M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      mw[w] = all[(w * 16 + r) * (D + 2) + D];
      M = fmaxf(M, mw[w]);
    }
    float value;
    if (c == D) {
      value = M;
    } else {  // accumulator columns and the mass column scale alike
      value = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w)
        value += mw[w] == -INFINITY ? 0.f : all[(w * 16 + r) * (D + 2) + c] * exp2f(mw[w] - M);
    }
    partials[((static_cast<size_t>(b) * q_heads + head0 + r) * n_splits + split) * (D + 2) + c] = value;
  }
}

// out[b, head, :] = sum_i acc_i 2^(m_i - M) / sum_i l_i 2^(m_i - M); one block per (b, head).
// Branch-free and in chunks of 8 parts, so that a chunk's loads are all in flight together.
template <int D>
__global__ void attention_merge_kernel(const float* __restrict__ partials,
                                       __nv_bfloat16* __restrict__ out, int n_parts) {
  pdl_trigger();  // a small kernel: let the next one start (and prefetch its weights) right away
  pdl_wait();
  const float* src = partials + static_cast<size_t>(blockIdx.x) * n_parts * (D + 2);
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float M = -INFINITY;
    for (int i0 = 0; i0 < n_parts; i0 += 8) {
      float mi[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) mi[u] = i0 + u < n_parts ? src[(i0 + u) * (D + 2) + D] : -INFINITY;
#pragma unroll
      for (int u = 0; u < 8; ++u) M = fmaxf(M, mi[u]);
    }
    float acc = 0.f, mass = 0.f;
    for (int i0 = 0; i0 < n_parts; i0 += 8) {
      float mi[8], ai[8], li[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const bool in = i0 + u < n_parts;
        const float* part_src = src + (in ? i0 + u : 0) * (D + 2);
        mi[u] = in ? part_src[D] : -INFINITY;
        ai[u] = part_src[d];
        li[u] = part_src[D + 1];
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {  // a part that saw no key has max -inf and weight 0
        const float w = mi[u] == -INFINITY ? 0.f : exp2f(mi[u] - M);
        acc = fmaf(ai[u], w, acc);
        mass = fmaf(li[u], w, mass);
      }
    }
    out[static_cast<size_t>(blockIdx.x) * D + d] = __float2bfloat16_rn(acc / mass);
  }
}

template <int D> int prefill_launch(const void* q, const void* k, const void* v, void* out,
                                    const int* cu_seqlens, int seqs, int max_seq_len, int q_heads,
                                    int kv_heads, float scale, int window, cudaStream_t stream) {
  const int smem = 4 * kTile * (D + 8) * 2;
  auto kernel = attention_prefill_tiled_kernel<D>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (seqs > 65535 || (max_seq_len + kTile - 1) / kTile > 65535) return LRM_UNSUPPORTED;
  const dim3 grid(q_heads, seqs, (max_seq_len + kTile - 1) / kTile);
  LRM_LAUNCH(kernel, grid, kThreads, smem, stream, static_cast<const __nv_bfloat16*>(q),
             static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v),
             static_cast<__nv_bfloat16*>(out), cu_seqlens, q_heads, kv_heads,
             scale * 1.4426950408889634f, window);
  return 0;
}

template <int D> int extend_launch(const void* q, const void* k_pages, const void* v_pages, void* out,
                                   const int* cu_seqlens, const int* page_table, int table_stride,
                                   const int* slots, const int* kv_lens, int seqs, int max_seq_len,
                                   int q_heads, int kv_heads, float scale, int window, cudaStream_t stream) {
  const int smem = 4 * kTile * (D + 8) * 2;
  auto kernel = attention_extend_tiled_kernel<D>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (seqs > 65535 || (max_seq_len + kTile - 1) / kTile > 65535) return LRM_UNSUPPORTED;
  const dim3 grid(q_heads, seqs, (max_seq_len + kTile - 1) / kTile);
  LRM_LAUNCH(kernel, grid, kThreads, smem, stream, static_cast<const __nv_bfloat16*>(q),
             static_cast<const __nv_bfloat16*>(k_pages), static_cast<const __nv_bfloat16*>(v_pages),
             static_cast<__nv_bfloat16*>(out), cu_seqlens, page_table, table_stride, slots, kv_lens,
             q_heads, kv_heads, scale * 1.4426950408889634f, window);
  return 0;
}

template <int D> int decode_launch(const void* q, const void* k_pages, const void* v_pages,
                                   float* partials, void* out, const int* page_table,
                                   int table_stride, const int* slots, const int* kv_lens, int seqs,
                                   int q_heads, int kv_heads, float scale, int window, int n_splits,
                                   cudaStream_t stream) {
  const int smem = 4 * kTile * (D + 8) * 2;
  auto kernel = attention_decode_tiled_kernel<D>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return static_cast<int>(e);
  const int group = q_heads / kv_heads, row_groups = (group + 15) / 16;
  const dim3 grid(seqs * kv_heads * row_groups, n_splits);
  LRM_LAUNCH(kernel, grid, kThreads, smem, stream, static_cast<const __nv_bfloat16*>(q),
             static_cast<const __nv_bfloat16*>(k_pages), static_cast<const __nv_bfloat16*>(v_pages),
             partials, page_table, table_stride, slots, kv_lens, q_heads, kv_heads, row_groups,
             scale * 1.4426950408889634f, window, n_splits);
  LRM_LAUNCH(attention_merge_kernel<D>, seqs * q_heads, D <= 64 ? 64 : 128, 0, stream, partials,
             static_cast<__nv_bfloat16*>(out), n_splits);
  return 0;
}

}  // namespace

// Head sizes the tiled kernels take; the caller falls back to the row-wise kernel otherwise.
LRM_API int lrm_attention_tiled_supports(int head_dim, int page_size) {
  return (head_dim == 32 || head_dim == 64 || head_dim == 128) && page_size == kTile ? 1 : 0;
}

LRM_API int lrm_attention_prefill_tiled(const void* q, const void* k, const void* v, void* out,
                                        const int* cu_seqlens, int seqs, int max_seq_len,
                                        int q_heads, int kv_heads, int d, float scale, int window,
                                        cudaStream_t stream) {
  if (seqs <= 0 || max_seq_len <= 0) return 0;
  if (q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads != 0) return LRM_BAD_ARGUMENT;
  if (q_heads > 65535 || seqs > 65535) return LRM_UNSUPPORTED;
  switch (d) {
    case 32: return prefill_launch<32>(q, k, v, out, cu_seqlens, seqs, max_seq_len, q_heads, kv_heads, scale, window, stream);
    case 64: return prefill_launch<64>(q, k, v, out, cu_seqlens, seqs, max_seq_len, q_heads, kv_heads, scale, window, stream);
    case 128: return prefill_launch<128>(q, k, v, out, cu_seqlens, seqs, max_seq_len, q_heads, kv_heads, scale, window, stream);
    default: return LRM_UNSUPPORTED;
  }
}

// q, out: [tokens, q_heads, d] packed bfloat16 (sequence b's rows are cu_seqlens[b] ..
// cu_seqlens[b+1] - 1, at most max_seq_len of them); the cache holds every sequence's keys up to
// kv_lens[b] - 1, the step's own included.
LRM_API int lrm_attention_extend_tiled(const void* q, const void* k_pages, const void* v_pages, void* out,
                                       const int* cu_seqlens, const int* page_table, int table_stride,
                                       const int* slots, const int* kv_lens, int seqs, int max_seq_len,
                                       int q_heads, int kv_heads, int d, int page_size, float scale,
                                       int window, cudaStream_t stream) {
  if (seqs <= 0 || max_seq_len <= 0) return 0;
  if (q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads != 0) return LRM_BAD_ARGUMENT;
  if (q_heads > 65535 || seqs > 65535 || page_size != kTile) return LRM_UNSUPPORTED;
  switch (d) {
    case 32: return extend_launch<32>(q, k_pages, v_pages, out, cu_seqlens, page_table, table_stride, slots, kv_lens, seqs, max_seq_len, q_heads, kv_heads, scale, window, stream);
    case 64: return extend_launch<64>(q, k_pages, v_pages, out, cu_seqlens, page_table, table_stride, slots, kv_lens, seqs, max_seq_len, q_heads, kv_heads, scale, window, stream);
    case 128: return extend_launch<128>(q, k_pages, v_pages, out, cu_seqlens, page_table, table_stride, slots, kv_lens, seqs, max_seq_len, q_heads, kv_heads, scale, window, stream);
    default: return LRM_UNSUPPORTED;
  }
}

// Scratch: `partials`, seqs * q_heads * n_splits * (d + 2) floats (contents do not matter).
// Launches that share scratch must not overlap on the GPU.
LRM_API int lrm_attention_decode_tiled(const void* q, const void* k_pages, const void* v_pages,
                                       float* partials, void* out, const int* page_table,
                                       int table_stride, const int* slots, const int* kv_lens,
                                       int seqs, int q_heads, int kv_heads, int d, int page_size,
                                       float scale, int window, int n_splits, cudaStream_t stream) {
  if (seqs <= 0) return 0;
  if (q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads != 0 || n_splits <= 0 ||
      partials == nullptr)
    return LRM_BAD_ARGUMENT;
  if (page_size != kTile || n_splits > 65535) return LRM_UNSUPPORTED;
  switch (d) {
    case 32: return decode_launch<32>(q, k_pages, v_pages, partials, out, page_table, table_stride, slots, kv_lens, seqs, q_heads, kv_heads, scale, window, n_splits, stream);
    case 64: return decode_launch<64>(q, k_pages, v_pages, partials, out, page_table, table_stride, slots, kv_lens, seqs, q_heads, kv_heads, scale, window, n_splits, stream);
    case 128: return decode_launch<128>(q, k_pages, v_pages, partials, out, page_table, table_stride, slots, kv_lens, seqs, q_heads, kv_heads, scale, window, n_splits, stream);
    default: return LRM_UNSUPPORTED;
  }
}

// --------------------------------------------------------------------------- no-allocation variant
// See attention_static_scratch.h: the same decode attention with its partials in a static
// device array, for callers that cannot allocate. No counterpart in the reference.
#include "attention_static_scratch.h"

#include <mutex>

namespace {
constexpr int kStaticScratchFloats = 1 << 20;  // 4 MiB per device that loads the library
constexpr int kMaxDevices = 64;
// In host code this name is only a handle for cudaGetSymbolAddress, never a device pointer.
static __device__ __align__(256) float g_static_partials[kStaticScratchFloats];
float* g_static_partials_address[kMaxDevices] = {};
std::mutex g_static_partials_mutex;

// Device address of the array on the current device; looked up once per device.
int static_partials(float** address) {
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (device < 0 || device >= kMaxDevices) return LRM_UNSUPPORTED;
  std::lock_guard<std::mutex> guard(g_static_partials_mutex);
  if (g_static_partials_address[device] == nullptr) {
    void* found = nullptr;
    e = cudaGetSymbolAddress(&found, g_static_partials);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (found == nullptr) return LRM_UNSUPPORTED;
    g_static_partials_address[device] = static_cast<float*>(found);
  }
  *address = g_static_partials_address[device];
  return 0;
}
}  // namespace

LRM_API int lrm_attention_static_scratch_floats(void) { return kStaticScratchFloats; }

LRM_API int lrm_attention_decode_tiled_static_scratch(const void* q, const void* k_pages,
                                                      const void* v_pages, void* out,
                                                      const int* page_table, int table_stride,
                                                      const int* slots, const int* kv_lens, int seqs,
                                                      int q_heads, int kv_heads, int head_dim,
                                                      int page_size, float scale, int window,
                                                      int n_splits, cudaStream_t stream) {
  if (seqs <= 0) return 0;
  if (q_heads <= 0 || kv_heads <= 0 || head_dim <= 0 || n_splits <= 0) return LRM_BAD_ARGUMENT;
  const long long needed =
      static_cast<long long>(seqs) * q_heads * n_splits * (static_cast<long long>(head_dim) + 2);
  if (needed > kStaticScratchFloats) return LRM_SCRATCH_EXCEEDED;
  float* partials = nullptr;
  const int status = static_partials(&partials);
  if (status != 0) return status;
  // Every (sequence, head, split) partial is written by the first kernel before the second
  // reads it, so nothing in the array needs clearing between calls.
  return lrm_attention_decode_tiled(q, k_pages, v_pages, partials, out, page_table, table_stride,
                                    slots, kv_lens, seqs, q_heads, kv_heads, head_dim, page_size,
                                    scale, window, n_splits, stream);
}

LRM_API const char* lrm_attention_static_scratch_error(int code) {
  switch (code) {
    case 0: return "ok";
    case LRM_SCRATCH_EXCEEDED:
      return "seqs * q_heads * n_splits * (head_dim + 2) floats of partials do not fit the 4 MiB static "
             "scratch: use fewer splits or a smaller batch";
    case LRM_BAD_ARGUMENT: return "bad argument";
    case LRM_UNSUPPORTED: return "head size, page size or device not supported by the tiled decode kernel";
    default: return "CUDA error (the code is a cudaError_t)";
  }
}
