// The epilogues of the tensor-core products, applied to 32 columns of one accumulator row at a time
// (shared by the single-CTA kernel and the kernel that runs pairs of CTAs):
//   0 store bfloat16, 1 store float32, 2 add into float32 in place (residual stream),
//   3 SiLU gate over alternating blocks of 8 gate / 8 up columns, 4 store float32 (a K slice's plane).
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

}  // namespace
