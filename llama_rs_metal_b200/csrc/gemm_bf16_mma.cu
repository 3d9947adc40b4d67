// bfloat16 matrix product with float32 accumulation on the warp-level tensor
// path (mma.sync m16n8k16): C[M,N] = X[M,K] . W[N,K]^T for any M, N, K.
// This is the kernel for shapes the TMA/tcgen05 kernels refuse (K not a
// multiple of 8, tiny matrices) and the yardstick they are checked against.
//
// Epilogues (what is done with the float32 accumulator):
//   0  store bfloat16                 C[M,N]
//   1  store float32                  C[M,N]
//   2  add into float32 in place      C[M,N] += acc      (residual stream)
//   3  SiLU-gate: the N rows of W come in alternating blocks of 8 gate rows
//      and 8 up rows; out[M, N/2] = silu(gate) * up as bfloat16
//      (reference: crates/metal-backend/src/shaders/elementwise.metal:8-17).
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 32, PAD = 8;

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4],
                                               const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

__device__ __forceinline__ float silu_f32(float g) { return g / (1.0f + expf(-g)); }

// Copy a [rows x BK] tile of a row-major [total_rows, K] matrix into shared
// memory, zero-filling outside the matrix. 16-byte loads when the row pitch
// allows it, element loads otherwise.
__device__ __forceinline__ void load_tile(__nv_bfloat16 (*dst)[BK + PAD],
                                          const __nv_bfloat16* __restrict__ src, int row0,
                                          int total_rows, int k0, int K, bool vector_ok) {
  for (int idx = threadIdx.x; idx < BM * (BK / 8); idx += blockDim.x) {
    const int r = idx / (BK / 8), c = (idx % (BK / 8)) * 8;
    const int gr = row0 + r, gk = k0 + c;
    uint4 val = make_uint4(0u, 0u, 0u, 0u);
    if (gr < total_rows) {
      const __nv_bfloat16* p = src + static_cast<size_t>(gr) * K + gk;
      if (vector_ok && gk + 8 <= K) {
        val = *reinterpret_cast<const uint4*>(p);
      } else {
        __align__(16) __nv_bfloat16 tmp[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) tmp[e] = gk + e < K ? p[e] : __float2bfloat16_rn(0.f);
        val = *reinterpret_cast<const uint4*>(tmp);
      }
    }
    *reinterpret_cast<uint4*>(&dst[r][c]) = val;
  }
}

__global__ __launch_bounds__(128) void gemm_bf16_mma_kernel(const __nv_bfloat16* __restrict__ X,
                                                            const __nv_bfloat16* __restrict__ W,
                                                            void* __restrict__ C, int M, int N,
                                                            int K, int mode, int vector_ok) {
  __shared__ __align__(16) __nv_bfloat16 Xs[BM][BK + PAD];
  __shared__ __align__(16) __nv_bfloat16 Ws[BN][BK + PAD];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int wm = (warp >> 1) * 32, wn = (warp & 1) * 32;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[2][4][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    load_tile(Xs, X, m0, M, k0, K, vector_ok != 0);
    load_tile(Ws, W, n0, N, k0, K, vector_ok != 0);
    __syncthreads();
#pragma unroll
    for (int ks = 0; ks < BK; ks += 16) {
      uint32_t a[2][4], b[4][2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int r = wm + i * 16 + g;
        a[i][0] = *reinterpret_cast<const uint32_t*>(&Xs[r][ks + 2 * t]);
        a[i][1] = *reinterpret_cast<const uint32_t*>(&Xs[r + 8][ks + 2 * t]);
        a[i][2] = *reinterpret_cast<const uint32_t*>(&Xs[r][ks + 2 * t + 8]);
        a[i][3] = *reinterpret_cast<const uint32_t*>(&Xs[r + 8][ks + 2 * t + 8]);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = wn + j * 8 + g;
        b[j][0] = *reinterpret_cast<const uint32_t*>(&Ws[n][ks + 2 * t]);
        b[j][1] = *reinterpret_cast<const uint32_t*>(&Ws[n][ks + 2 * t + 8]);
      }
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) mma_bf16_16816(acc[i][j], a[i], b[j]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 2; ++i) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int row = m0 + wm + i * 16 + g + half * 8;
      if (row >= M) continue;
      if (mode == 3) {
#pragma unroll
        for (int j = 0; j < 4; j += 2) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int col = n0 + wn + j * 8 + 2 * t + e;  // a gate column; its up column is col + 8
            if (col + 8 >= N) continue;
            const float gate = acc[i][j][half * 2 + e], up = acc[i][j + 1][half * 2 + e];
            const int out_col = (col / 16) * 8 + (col % 8);
            static_cast<__nv_bfloat16*>(C)[static_cast<size_t>(row) * (N / 2) + out_col] =
                __float2bfloat16_rn(silu_f32(gate) * up);
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int col = n0 + wn + j * 8 + 2 * t + e;
            if (col >= N) continue;
            const float v = acc[i][j][half * 2 + e];
            const size_t o = static_cast<size_t>(row) * N + col;
            if (mode == 0) static_cast<__nv_bfloat16*>(C)[o] = __float2bfloat16_rn(v);
            else if (mode == 1) static_cast<float*>(C)[o] = v;
            else static_cast<float*>(C)[o] += v;
          }
        }
      }
    }
  }
}
}  // namespace

LRM_API int lrm_gemm_bf16_mma(const void* X, const void* W, void* C, int M, int N, int K, int mode,
                              cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || mode < 0 || mode > 3) return LRM_BAD_ARGUMENT;
  if (mode == 3 && N % 16 != 0) return LRM_BAD_ARGUMENT;
  const dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return LRM_UNSUPPORTED;
  const bool aligned = (reinterpret_cast<uintptr_t>(X) % 16 == 0) &&
                       (reinterpret_cast<uintptr_t>(W) % 16 == 0) && (K % 8 == 0);
  gemm_bf16_mma_kernel<<<grid, 128, 0, stream>>>(static_cast<const __nv_bfloat16*>(X),
                                                 static_cast<const __nv_bfloat16*>(W), C, M, N, K,
                                                 mode, aligned ? 1 : 0);
  LRM_LAUNCH_CHECK();
  return 0;
}
