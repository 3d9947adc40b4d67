// Device helpers shared by the attention kernels on the warp-level tensor path
// (mma.sync m16n8k16, ldmatrix, cp.async): 64-key tiles with rows padded by 8 elements,
// float32 scores in the log2 domain, streaming softmax.
#pragma once
#include "common.cuh"

namespace {

constexpr int kTile = 64;     // keys per tile (= the cache's page size)
constexpr int kThreads = 128;  // 4 warps

__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3,
                                        const void* p) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                              uint32_t& r3, const void* p) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(a));
}
// 16-byte asynchronous copy; `bytes` = 0 writes zeros and reads nothing.
__device__ __forceinline__ void cp_async16(void* dst, const void* src, int bytes) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Copy `rows` x D bfloat16 (row pitch `pitch` elements in global memory) into a
// padded shared tile; rows >= valid_rows are zero-filled.
template <int D>
__device__ __forceinline__ void load_tile(__nv_bfloat16* dst, const __nv_bfloat16* src, size_t pitch,
                                          int valid_rows) {
  constexpr int STRIDE = D + 8, CHUNKS = D / 8;
  for (int idx = threadIdx.x; idx < kTile * CHUNKS; idx += kThreads) {
    const int r = idx / CHUNKS, c = idx % CHUNKS;
    const bool ok = r < valid_rows;
    cp_async16(dst + r * STRIDE + c * 8, ok ? src + r * pitch + c * 8 : src, ok ? 16 : 0);
  }
}

// The same for one page of the cache (64 rows of D elements, contiguous): a thread's copies differ
// by constants, and a page whose rows all count needs no test per row. Rows outside
// [first_row, valid_rows) are zero-filled: behind a sequence's end, and before a window's first
// key, the cache may hold anything (rows never written, even NaN bit patterns).
template <int D>
__device__ __forceinline__ void load_page(__nv_bfloat16* dst, const __nv_bfloat16* src, int valid_rows,
                                          int first_row = 0) {
  constexpr int STRIDE = D + 8, CHUNKS = D / 8, ROWS = kThreads / CHUNKS;  // rows covered per pass
  const int r0 = threadIdx.x / CHUNKS, c8 = (threadIdx.x % CHUNKS) * 8;
  const __nv_bfloat16* s = src + r0 * D + c8;
  __nv_bfloat16* d = dst + r0 * STRIDE + c8;
  if (valid_rows >= kTile && first_row <= 0) {
#pragma unroll
    for (int i = 0; i < kTile / ROWS; ++i) cp_async16(d + i * ROWS * STRIDE, s + i * ROWS * D, 16);
  } else {
#pragma unroll
    for (int i = 0; i < kTile / ROWS; ++i) {
      const bool ok = r0 + i * ROWS < valid_rows && r0 + i * ROWS >= first_row;
      cp_async16(d + i * ROWS * STRIDE, ok ? s + i * ROWS * D : src, ok ? 16 : 0);
    }
  }
}

// Query fragments of 16 rows x D from global memory: row r lives at base + r * pitch.
template <int D>
__device__ __forceinline__ void load_q(uint32_t (&qa)[D / 16][4], const __nv_bfloat16* base,
                                       size_t pitch, int valid_rows) {
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = g + 8 * half;
#pragma unroll
      for (int hi = 0; hi < 2; ++hi) {
        uint32_t v = 0u;
        if (r < valid_rows)
          v = *reinterpret_cast<const uint32_t*>(base + r * pitch + 16 * ks + 8 * hi + 2 * t);
        qa[ks][half + 2 * hi] = v;
      }
    }
  }
}

// s[nt] (16 x 8) += Q (16 x D) . K^T for the 8-key tiles nt of `keys` (rows of a padded tile).
template <int D, int NT>
__device__ __forceinline__ void scores(float (&s)[NT][4], const uint32_t (&qa)[D / 16][4],
                                       const __nv_bfloat16* keys) {
  constexpr int STRIDE = D + 8;
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
    for (int ks = 0; ks < D / 16; ks += 2) {
      uint32_t b0, b1, b2, b3;
      ldsm_x4(b0, b1, b2, b3, keys + (8 * nt + (lane & 7)) * STRIDE + 16 * ks + 8 * (lane >> 3));
      mma16816(s[nt], qa[ks], b0, b1);
      mma16816(s[nt], qa[ks + 1], b2, b3);
    }
  }
}

// o (16 x D) += P (16 x 16*KK keys) . V, P given as score tiles already turned into probabilities.
template <int D, int NT>
__device__ __forceinline__ void weighted_values(float (&o)[D / 8][4], const float (&p)[NT][4],
                                                const __nv_bfloat16* values) {
  constexpr int STRIDE = D + 8;
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int kk = 0; kk < NT / 2; ++kk) {
    uint32_t pa[4];
    pa[0] = pack_bf16(p[2 * kk][0], p[2 * kk][1]);
    pa[1] = pack_bf16(p[2 * kk][2], p[2 * kk][3]);
    pa[2] = pack_bf16(p[2 * kk + 1][0], p[2 * kk + 1][1]);
    pa[3] = pack_bf16(p[2 * kk + 1][2], p[2 * kk + 1][3]);
#pragma unroll
    for (int dn = 0; dn < D / 8; dn += 2) {
      uint32_t b0, b1, b2, b3;
      ldsm_x4_trans(b0, b1, b2, b3,
                    values + (16 * kk + (lane & 7) + 8 * ((lane >> 3) & 1)) * STRIDE + 8 * dn +
                        8 * (lane >> 4));
      mma16816(o[dn], pa, b0, b1);
      mma16816(o[dn + 1], pa, b2, b3);
    }
  }
}

// 2^x on the special-function unit (x <= 0 here; results below the normal range flush to zero).
__device__ __forceinline__ float exp2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// One streaming-softmax update of rows g and g+8 with NT score tiles (already masked to -inf
// where a key is not visible). m, l: running max (log2 domain) and this thread's share of the mass.
// HALVES = 1 leaves rows g+8 alone (a caller whose rows 8..15 are padding).
template <int D, int NT, int HALVES = 2>
__device__ __forceinline__ void softmax_update(float (&s)[NT][4], float (&o)[D / 8][4], float (&m)[2],
                                               float (&l)[2]) {
#pragma unroll
  for (int half = 0; half < HALVES; ++half) {
    float mx = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) mx = fmaxf(mx, fmaxf(s[nt][2 * half], s[nt][2 * half + 1]));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m[half], mx);
    const float m_use = m_new == -INFINITY ? 0.f : m_new;  // a row with no visible key yet
    const float alpha = exp2_fast(m[half] - m_use);
    float sum = 0.f;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      s[nt][2 * half] = exp2_fast(s[nt][2 * half] - m_use);
      s[nt][2 * half + 1] = exp2_fast(s[nt][2 * half + 1] - m_use);
      sum += s[nt][2 * half] + s[nt][2 * half + 1];
    }
    l[half] = l[half] * alpha + sum;
    m[half] = m_new;
#pragma unroll
    for (int dn = 0; dn < D / 8; ++dn) {
      o[dn][2 * half] *= alpha;
      o[dn][2 * half + 1] *= alpha;
    }
  }
  if (HALVES == 1) {  // rows g+8 are padding: their probabilities must not reach the products
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) s[nt][2] = s[nt][3] = 0.f;
  }
}

}  // namespace
