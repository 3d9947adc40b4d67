// RMSNorm over rows of the float32 residual stream:
//   inv = 1 / sqrt(mean(x^2) + eps);  y = (x * inv) * w
// (reference: crates/metal-backend/src/shaders/elementwise.metal:31-46).
// The sum of squares is float32 in a fixed order; the output is float32 or
// bfloat16. Optional fusions, all in the same pass over the row:
//  * `rows`: normalize only the listed rows (the head runs on wanted rows);
//  * `partials`: `n_partials` float32 [T,h] slices that are first added, in
//    slice order, into the residual row, which is written back (this folds a
//    split-K projection's partial sums and the residual add into the norm).
#include "common.cuh"

template <typename W, typename O>
__global__ void rms_norm_kernel(float* __restrict__ x, const W* __restrict__ w, O* __restrict__ out,
                                const int* __restrict__ rows, const float* __restrict__ partials,
                                int n_partials, size_t partial_stride, int hidden, float eps) {
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  const size_t src = static_cast<size_t>(rows ? rows[r] : r) * hidden;
  float* xr = x + src;
  O* yr = out + static_cast<size_t>(r) * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = xr[i];
    if (n_partials > 0) {
      for (int p = 0; p < n_partials; ++p) v += partials[p * partial_stride + src + i];
      xr[i] = v;
    }
    ss = fmaf(v, v, ss);
  }
  const float total = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(total / static_cast<float>(hidden) + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    yr[i] = from_f32<O>((xr[i] * inv) * to_f32(w[i]));
}

template <typename W, typename O>
static void launch_norm(float* x, const void* w, void* out, const int* rows, const float* partials,
                        int n_partials, size_t partial_stride, int n_rows, int hidden, float eps,
                        cudaStream_t stream) {
  const int threads = hidden >= 1024 ? 256 : (hidden >= 256 ? 128 : 32);
  rms_norm_kernel<W, O><<<n_rows, threads, 0, stream>>>(
      x, static_cast<const W*>(w), static_cast<O*>(out), rows, partials, n_partials, partial_stride,
      hidden, eps);
}

LRM_API int lrm_rms_norm(float* x, const void* w, int w_dtype, void* out, int out_dtype,
                         const int* rows, const float* partials, int n_partials,
                         long long partial_stride, int n_rows, int hidden, float eps,
                         cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (hidden <= 0 || !(eps > 0.f)) return LRM_BAD_ARGUMENT;
  if (rows != nullptr && n_partials > 0) return LRM_BAD_ARGUMENT;  // a gathered row is not written back
  const size_t ps = static_cast<size_t>(partial_stride);
#define LRM_NORM(WT, OT) launch_norm<WT, OT>(x, w, out, rows, partials, n_partials, ps, n_rows, hidden, eps, stream)
  if (w_dtype == LRM_F32 && out_dtype == LRM_F32) LRM_NORM(float, float);
  else if (w_dtype == LRM_F32 && out_dtype == LRM_BF16) LRM_NORM(float, __nv_bfloat16);
  else if (w_dtype == LRM_BF16 && out_dtype == LRM_F32) LRM_NORM(__nv_bfloat16, float);
  else if (w_dtype == LRM_BF16 && out_dtype == LRM_BF16) LRM_NORM(__nv_bfloat16, __nv_bfloat16);
  else return LRM_BAD_ARGUMENT;
#undef LRM_NORM
  LRM_LAUNCH_CHECK();
  return 0;
}
