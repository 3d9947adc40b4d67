// True 32-bit matrix product on the CUDA cores: C[M,N] = X[M,K] . W[N,K]^T.
// W is a Linear weight as stored ([out][in]); every product and sum is an
// IEEE float32 fused multiply-add, with no tensor-core or reduced-precision
// mode anywhere. Each output element is accumulated over k = 0..K-1 in
// ascending order by one thread, so its value does not depend on M, on the
// tile it falls in, or on what else is in the batch.
// (Reference role: the F32 simdgroup GEMM/GEMV family,
// crates/metal-backend/src/shaders/matrix.metal:10-37,236-282.)
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16;

// mode 0: C = acc;  mode 1: C += acc (the residual add folded into the epilogue)
__global__ __launch_bounds__(256) void gemm_f32_kernel(const float* __restrict__ X,
                                                       const float* __restrict__ W,
                                                       float* __restrict__ C, int M, int N, int K,
                                                       int mode) {
  __shared__ float Xs[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = tid + i * 256, r = idx >> 4, c = idx & 15;
      const int gk = k0 + c;
      const int gm = m0 + r, gn = n0 + r;
      Xs[c][r] = (gm < M && gk < K) ? X[static_cast<size_t>(gm) * K + gk] : 0.f;
      Ws[c][r] = (gn < N && gk < K) ? W[static_cast<size_t>(gn) * K + gk] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = Xs[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn >= N) continue;
      float* dst = C + static_cast<size_t>(gm) * N + gn;
      *dst = mode == 1 ? *dst + acc[i][j] : acc[i][j];
    }
  }
}
}  // namespace

LRM_API int lrm_gemm_f32(const float* X, const float* W, float* C, int M, int N, int K, int mode,
                         cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (mode != 0 && mode != 1)) return LRM_BAD_ARGUMENT;
  const dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return LRM_UNSUPPORTED;
  gemm_f32_kernel<<<grid, 256, 0, stream>>>(X, W, C, M, N, K, mode);
  LRM_LAUNCH_CHECK();
  return 0;
}
