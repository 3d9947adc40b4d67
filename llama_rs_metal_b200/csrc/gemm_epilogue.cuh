// The epilogues of the tensor-core products, applied to 32 columns of one accumulator row at a time
// (shared by the single-CTA kernel and the kernel that runs pairs of CTAs):
//   0 store bfloat16, 1 store float32, 2 add into float32 in place (residual stream),
//   3 SiLU gate over alternating blocks of 8 gate / 8 up columns, 4 store float32 (a K slice's plane),
// and epilogue 5, which works on whole heads of a fused q|k|v projection (store_heads).
#pragma once
#include "umma.cuh"

namespace {

__device__ __forceinline__ float silu_f32(float g) { return g / (1.0f + expf(-g)); }

// The epilogue of one 32-column piece of an accumulator row held in registers.
__device__ __forceinline__ void store_piece(const uint32_t (&r)[32], void* __restrict__ out, int m, int n,
                                            int M, int N, int mode) {
  if (m >= M || n >= N) return;
  const bool whole = n + 32 <= N;
  if (mode == 3) {
    // [8 gate | 8 up | 8 gate | 8 up] -> 16 gated values
    __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(out) + static_cast<size_t>(m) * (N >> 1) + (n >> 1);
    uint32_t packed[8];
#pragma unroll
    for (int i = 0; i < 16; i += 2) {
      const int a = (i >> 3) * 16 + (i & 7);
      const float v0 = silu_f32(__uint_as_float(r[a])) * __uint_as_float(r[a + 8]);
      const float v1 = silu_f32(__uint_as_float(r[a + 1])) * __uint_as_float(r[a + 9]);
      packed[i >> 1] = pack_bf16(v0, v1);
    }
    if (whole) {
      *reinterpret_cast<uint4*>(dst) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
      *reinterpret_cast<uint4*>(dst + 8) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
    } else {
      const __nv_bfloat16* vals = reinterpret_cast<const __nv_bfloat16*>(packed);
      for (int i = 0; i < 16 && n + (i >> 3) * 16 + 8 + (i & 7) < N; ++i) dst[i] = vals[i];
    }
  } else if (mode == 0) {
    __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(out) + static_cast<size_t>(m) * N + n;
    if (whole && (N & 7) == 0) {
#pragma unroll
      for (int i = 0; i < 32; i += 8)
        *reinterpret_cast<uint4*>(dst + i) = make_uint4(
            pack_bf16(__uint_as_float(r[i]), __uint_as_float(r[i + 1])),
            pack_bf16(__uint_as_float(r[i + 2]), __uint_as_float(r[i + 3])),
            pack_bf16(__uint_as_float(r[i + 4]), __uint_as_float(r[i + 5])),
            pack_bf16(__uint_as_float(r[i + 6]), __uint_as_float(r[i + 7])));
    } else {
      for (int i = 0; i < 32 && n + i < N; ++i) dst[i] = __float2bfloat16_rn(__uint_as_float(r[i]));
    }
  } else {
    float* dst = static_cast<float*>(out) + static_cast<size_t>(m) * N + n;
    if (whole && (N & 3) == 0) {
#pragma unroll
      for (int i = 0; i < 32; i += 4) {
        float4 v = make_float4(__uint_as_float(r[i]), __uint_as_float(r[i + 1]), __uint_as_float(r[i + 2]),
                               __uint_as_float(r[i + 3]));
        // Adding goes through a vector reduction in L2 (no value comes back, so the thread does
        // not wait for the old contents). Each element gets exactly one add per launch, so the
        // result is as deterministic as a read-modify-write.
        if (mode == 2) atomicAdd(reinterpret_cast<float4*>(dst + i), v);
        else *reinterpret_cast<float4*>(dst + i) = v;
      }
    } else {
      for (int i = 0; i < 32 && n + i < N; ++i) {
        if (mode == 2) atomicAdd(dst + i, __uint_as_float(r[i]));
        else dst[i] = __uint_as_float(r[i]);
      }
    }
  }
}

// What epilogue 5 needs: the product is a prompt's fused q|k|v projection [T, (Hq + 2 Hk) d], and
// instead of storing it the epilogue rounds it to bfloat16, rotates q and k by their positions
// (split-half, the angles' cosines and sines from a table made once per step) and stores q, k
// and v packed for the prompt's own attention, and k and v into the paged cache as well: what
// rope_store.cu does in a launch of its own, with the same operations in the same order, so
// both ways give the same bits.
struct QkvArgs {
  __nv_bfloat16* q;          // [T, Hq, d]
  __nv_bfloat16* k;          // [T, Hk, d]
  __nv_bfloat16* v;          // [T, Hk, d]
  __nv_bfloat16* k_pages;    // [pages, Hk, page_size, d] or nullptr
  __nv_bfloat16* v_pages;
  const int* dest_rows;      // [T]: page * page_size + row of the token in the cache, < 0: not stored
  const float2* table;       // [T, d / 2] (cos, sin) of position * inverse frequency, or nullptr: no rotation
  int q_heads, kv_heads, head_dim, page_size;
};

__device__ __forceinline__ void store_32_bf16(__nv_bfloat16* dst, const uint32_t (&packed)[16]) {
#pragma unroll
  for (int i = 0; i < 16; i += 4)
    *reinterpret_cast<uint4*>(dst + 2 * i) = make_uint4(packed[i], packed[i + 1], packed[i + 2], packed[i + 3]);
}

// One accumulator row (token m) of a tile whose first column n0 is the first of a head and whose
// width BN is a whole number of heads: `tmem_row` addresses the row's first column in tensor
// memory. Every lane of the warp must call it (the loads are warp-wide); rows beyond M only load.
// Of the tile's heads this call takes those that begin in columns [first, last).
template <int BN>
__device__ __forceinline__ void store_heads(uint32_t tmem_row, int m, int n0, int M, int N, const QkvArgs& a,
                                            int first = 0, int last = BN) {
  const int d = a.head_dim, half = d >> 1;
  const bool live = m < M;
  const int dest = live && a.k_pages != nullptr ? a.dest_rows[m] : -1;
  const size_t page = dest >= 0 ? static_cast<size_t>(dest / a.page_size) : 0;
  const int in_page = dest >= 0 ? dest % a.page_size : 0;
  for (int c0 = first; c0 < last && n0 + c0 < N; c0 += d) {
    const int head = (n0 + c0) / d;
    const bool is_q = head < a.q_heads, is_v = head >= a.q_heads + a.kv_heads;
    const int kh = is_q ? 0 : head - a.q_heads - (is_v ? a.kv_heads : 0);
    __nv_bfloat16* packed_dst = is_q ? a.q + (static_cast<size_t>(m) * a.q_heads + head) * d
                                     : (is_v ? a.v : a.k) + (static_cast<size_t>(m) * a.kv_heads + kh) * d;
    __nv_bfloat16* cache_dst = (is_q || dest < 0) ? nullptr
        : (is_v ? a.v_pages : a.k_pages) + ((page * a.kv_heads + kh) * a.page_size + in_page) * d;
    if (is_v || a.table == nullptr) {
      for (int c = 0; c < d; c += 32) {
        uint32_t r[32];
        tmem_load32(tmem_row + c0 + c, r);
        if (live) {
          uint32_t packed[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) packed[i] = pack_bf16(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
          store_32_bf16(packed_dst + c, packed);
          if (cache_dst != nullptr) store_32_bf16(cache_dst + c, packed);
        }
      }
      continue;
    }
    for (int c = 0; c < half; c += 32) {  // columns c.. pair with columns half + c..
      uint32_t lo[32], hi[32];
      tmem_load32_async(tmem_row + c0 + c, lo);
      tmem_load32_async(tmem_row + c0 + half + c, hi);
      tmem_load_wait();
      tmem_pin(lo);
      tmem_pin(hi);
      if (live) {
        const float4* cs = reinterpret_cast<const float4*>(a.table + static_cast<size_t>(m) * half + c);
        uint32_t out_lo[16], out_hi[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {  // two pairs at a time: (cos, sin) of columns c + 2i and c + 2i + 1
          const float4 t = __ldg(cs + i);
          // the projection is rounded to bfloat16 first, as where it is stored before it is rotated
          const float xa0 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(lo[2 * i])));
          const float xa1 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(lo[2 * i + 1])));
          const float xb0 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(hi[2 * i])));
          const float xb1 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(hi[2 * i + 1])));
          out_lo[i] = pack_bf16(fmaf(xa0, t.x, -__fmul_rn(xb0, t.y)), fmaf(xa1, t.z, -__fmul_rn(xb1, t.w)));
          out_hi[i] = pack_bf16(fmaf(xa0, t.y, __fmul_rn(xb0, t.x)), fmaf(xa1, t.w, __fmul_rn(xb1, t.z)));
        }
        store_32_bf16(packed_dst + c, out_lo);
        store_32_bf16(packed_dst + half + c, out_hi);
        if (cache_dst != nullptr) {
          store_32_bf16(cache_dst + c, out_lo);
          store_32_bf16(cache_dst + half + c, out_hi);
        }
      }
    }
  }
}

}  // namespace
