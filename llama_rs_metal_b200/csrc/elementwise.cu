// Small elementwise kernels: the SiLU gate, the residual add and dtype casts.
#include "common.cuh"

// out[t, c] = silu(gate) * up where the 2I columns of `gate_up` come in
// alternating blocks of `block` gate columns and `block` up columns
// (block == I is plain [gate | up] concatenation).
// silu(g) = g / (1 + exp(-g))  (reference: elementwise.metal:8-17).
template <typename A>
__global__ void silu_mul_kernel(const A* __restrict__ gate_up, A* __restrict__ out, size_t total,
                                int inter, int block) {
  const size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (idx >= total) return;
  const size_t t = idx / inter;
  const int c = static_cast<int>(idx % inter);
  const size_t base = t * 2 * inter + static_cast<size_t>(c / block) * 2 * block + c % block;
  const float g = to_f32(gate_up[base]), u = to_f32(gate_up[base + block]);
  out[idx] = from_f32<A>(g / (1.0f + expf(-g)) * u);
}

template <typename D>
__global__ void add_inplace_kernel(float* __restrict__ x, const D* __restrict__ delta, size_t n) {
  const size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (idx < n) x[idx] += to_f32(delta[idx]);
}

// x += planes[0] + planes[1] + ... in plane order (the K slices of a product whose sum belongs
// to the residual stream), for a reader of the stream that cannot fold them itself.
__global__ void add_planes_kernel(float* __restrict__ x, const float* __restrict__ planes, int count,
                                  size_t n) {
  pdl_trigger();
  pdl_wait();
  const size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (idx >= n) return;
  float v = x[idx];
  for (int p = 0; p < count; ++p) v += planes[p * n + idx];
  x[idx] = v;
}

template <typename S, typename D>
__global__ void cast_kernel(const S* __restrict__ src, D* __restrict__ dst, size_t n) {
  const size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (idx < n) dst[idx] = from_f32<D>(to_f32(src[idx]));
}

static unsigned blocks_for(size_t n) { return static_cast<unsigned>((n + 255) / 256); }

LRM_API int lrm_silu_mul(const void* gate_up, void* out, int dtype, long long rows, int inter,
                         int block, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (inter <= 0 || block <= 0 || inter % block != 0) return LRM_BAD_ARGUMENT;
  const size_t total = static_cast<size_t>(rows) * inter;
  if (dtype == LRM_F32)
    silu_mul_kernel<float><<<blocks_for(total), 256, 0, stream>>>(
        static_cast<const float*>(gate_up), static_cast<float*>(out), total, inter, block);
  else if (dtype == LRM_BF16)
    silu_mul_kernel<__nv_bfloat16><<<blocks_for(total), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(gate_up), static_cast<__nv_bfloat16*>(out), total, inter,
        block);
  else
    return LRM_BAD_ARGUMENT;
  LRM_LAUNCH_CHECK();
  return 0;
}

LRM_API int lrm_add_inplace(float* x, const void* delta, int delta_dtype, long long n,
                            cudaStream_t stream) {
  if (n <= 0) return 0;
  if (delta_dtype == LRM_F32)
    add_inplace_kernel<float><<<blocks_for(n), 256, 0, stream>>>(x, static_cast<const float*>(delta), n);
  else if (delta_dtype == LRM_BF16)
    add_inplace_kernel<__nv_bfloat16><<<blocks_for(n), 256, 0, stream>>>(
        x, static_cast<const __nv_bfloat16*>(delta), n);
  else
    return LRM_BAD_ARGUMENT;
  LRM_LAUNCH_CHECK();
  return 0;
}

__global__ void scale_inplace_kernel(float* __restrict__ x, float factor, size_t n) {
  pdl_trigger();
  pdl_wait();
  const size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (idx < n) x[idx] *= factor;
}

LRM_API int lrm_scale_inplace(float* x, float factor, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (x == nullptr) return LRM_BAD_ARGUMENT;
  LRM_LAUNCH(scale_inplace_kernel, blocks_for(n), 256, 0, stream, x, factor, static_cast<size_t>(n));
  return 0;
}

LRM_API int lrm_add_planes(float* x, const float* planes, int count, long long n, cudaStream_t stream) {
  if (n <= 0 || count <= 0) return 0;
  if (x == nullptr || planes == nullptr) return LRM_BAD_ARGUMENT;
  LRM_LAUNCH(add_planes_kernel, blocks_for(n), 256, 0, stream, x, planes, count, static_cast<size_t>(n));
  return 0;
}

LRM_API int lrm_cast(const void* src, int src_dtype, void* dst, int dst_dtype, long long n,
                     cudaStream_t stream) {
  if (n <= 0) return 0;
  if (src_dtype == LRM_F32 && dst_dtype == LRM_BF16)
    cast_kernel<float, __nv_bfloat16><<<blocks_for(n), 256, 0, stream>>>(
        static_cast<const float*>(src), static_cast<__nv_bfloat16*>(dst), n);
  else if (src_dtype == LRM_BF16 && dst_dtype == LRM_F32)
    cast_kernel<__nv_bfloat16, float><<<blocks_for(n), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(src), static_cast<float*>(dst), n);
  else
    return LRM_BAD_ARGUMENT;
  LRM_LAUNCH_CHECK();
  return 0;
}

