// RMSNorm over rows of the float32 residual stream:
//   inv = 1 / sqrt(mean(x^2) + eps);  y = (x * inv) * w
// (reference: crates/metal-backend/src/shaders/elementwise.metal:31-46).
// The sum of squares is float32 in a fixed order; the output is float32 or
// bfloat16. Optional fusions, all in the same pass over the row:
//  * `rows`: normalize only the listed rows (the head runs on wanted rows); a gathered
//    row is never written back;
//  * `partials`: `n_partials` float32 [T,h] slices that are first added, in
//    slice order, into the residual row, which is written back (this folds a
//    split-K projection's partial sums and the residual add into the norm).
#include "common.cuh"

// PER: elements each thread keeps in registers (hidden <= PER * blockDim.x); the row is read
// once, the norm weight is fetched together with it so only one memory latency is exposed.
template <typename W, typename O, int PER>
__global__ void rms_norm_kernel(float* __restrict__ x, const W* __restrict__ w, O* __restrict__ out,
                                const int* __restrict__ rows, const float* __restrict__ partials,
                                int n_partials, size_t partial_stride, int hidden, float eps) {
  __shared__ float scratch[32];
  float wv[PER];
#pragma unroll
  for (int e = 0; e < PER; ++e) {  // weights do not depend on the kernel before this one
    const int i = threadIdx.x + e * blockDim.x;
    wv[e] = i < hidden ? to_f32(w[i]) : 0.f;
  }
  pdl_trigger();  // a small kernel: let the next one start (and prefetch its weights) right away
  pdl_wait();
  const int r = blockIdx.x;
  const size_t src = static_cast<size_t>(rows ? rows[r] : r) * hidden;
  float* xr = x + src;
  O* yr = out + static_cast<size_t>(r) * hidden;
  float xv[PER];
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < PER; ++e) {
    const int i = threadIdx.x + e * blockDim.x;
    float v = i < hidden ? xr[i] : 0.f;
    if (n_partials > 0 && i < hidden) {
      // eight slices' loads are in flight together; they are added in slice order
      for (int p0 = 0; p0 < n_partials; p0 += 8) {
        float part[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
          part[u] = p0 + u < n_partials ? partials[(p0 + u) * partial_stride + src + i] : 0.f;
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (p0 + u < n_partials) v += part[u];
      }
      if (rows == nullptr) xr[i] = v;  // the folded sum becomes the residual stream
    }
    xv[e] = v;
    ss = fmaf(v, v, ss);
  }
  const float total = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(total / static_cast<float>(hidden) + eps);
#pragma unroll
  for (int e = 0; e < PER; ++e) {
    const int i = threadIdx.x + e * blockDim.x;
    if (i < hidden) yr[i] = from_f32<O>((xv[e] * inv) * wv[e]);
  }
}

// The same with 16-byte accesses: a thread keeps PER4 groups of four consecutive elements.
// Needs hidden % 4 == 0 and 16-byte aligned rows.
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(lo.x, lo.y, hi.x, hi.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<uint32_t*>(&lo);
  raw.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = raw;
}

template <typename W, typename O, int PER4>
__global__ void rms_norm_vec_kernel(float* __restrict__ x, const W* __restrict__ w, O* __restrict__ out,
                                    const int* __restrict__ rows, const float* __restrict__ partials,
                                    int n_partials, size_t partial_stride, int hidden, float eps) {
  __shared__ float scratch[32];
  const int groups = hidden >> 2;
  float4 wv[PER4];
#pragma unroll
  for (int e = 0; e < PER4; ++e) {  // weights do not depend on the kernel before this one
    const int c = threadIdx.x + e * blockDim.x;
    wv[e] = c < groups ? load4(w + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  pdl_trigger();  // a small kernel: let the next one start (and prefetch its weights) right away
  pdl_wait();
  const int r = blockIdx.x;
  const size_t src = static_cast<size_t>(rows ? rows[r] : r) * hidden;
  float* xr = x + src;
  O* yr = out + static_cast<size_t>(r) * hidden;
  float4 xv[PER4];
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < PER4; ++e) {
    const int c = threadIdx.x + e * blockDim.x;
    float4 v = c < groups ? load4(xr + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
    if (n_partials > 0 && c < groups) {
      // eight slices' loads are in flight together; they are added in slice order
      for (int p0 = 0; p0 < n_partials; p0 += 8) {
        float4 part[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
          part[u] = p0 + u < n_partials ? load4(partials + (p0 + u) * partial_stride + src + 4 * c)
                                        : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (p0 + u < n_partials) v.x += part[u].x, v.y += part[u].y, v.z += part[u].z, v.w += part[u].w;
      }
      if (rows == nullptr) store4(xr + 4 * c, v);  // the folded sum becomes the residual stream
    }
    xv[e] = v;
    ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
  }
  const float total = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(total / static_cast<float>(hidden) + eps);
#pragma unroll
  for (int e = 0; e < PER4; ++e) {
    const int c = threadIdx.x + e * blockDim.x;
    if (c < groups)
      store4(yr + 4 * c, make_float4((xv[e].x * inv) * wv[e].x, (xv[e].y * inv) * wv[e].y,
                                     (xv[e].z * inv) * wv[e].z, (xv[e].w * inv) * wv[e].w));
  }
}

// The same row cut among the CTAs of a thread-block cluster (`ranks` of them, each with its share of
// the columns): for few rows with several slices to fold, where one CTA per row leaves most SMs
// idle and each of the busy ones reads (slices + 1) rows. Every CTA sends its share of the sum of
// squares into each peer's shared memory, one cluster barrier, and all add the shares in rank
// order, so every CTA of a row holds the same total. The order of the sum differs from the
// one-CTA kernel's: used where the output is bfloat16 only.
__device__ __forceinline__ uint32_t norm_cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

template <typename W, typename O, int PER4>
__global__ void rms_norm_cluster_kernel(float* __restrict__ x, const W* __restrict__ w, O* __restrict__ out,
                                        const int* __restrict__ rows, const float* __restrict__ partials,
                                        int n_partials, size_t partial_stride, int hidden, float eps, int ranks) {
  __shared__ float scratch[32];
  __shared__ float shares[8];  // shares[k]: rank k's part of the sum of squares, written by rank k
  const int rank = static_cast<int>(norm_cluster_rank()), r = blockIdx.x / ranks;
  const int groups = hidden >> 2, per_cta = (groups + ranks - 1) / ranks;
  const int g0 = rank * per_cta, g1 = min(groups, g0 + per_cta);
  float4 wv[PER4];
#pragma unroll
  for (int e = 0; e < PER4; ++e) {  // weights do not depend on the kernel before this one
    const int c = g0 + threadIdx.x + e * blockDim.x;
    wv[e] = c < g1 ? load4(w + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  pdl_trigger();
  pdl_wait();
  const size_t src = static_cast<size_t>(rows ? rows[r] : r) * hidden;
  float* xr = x + src;
  O* yr = out + static_cast<size_t>(r) * hidden;
  float4 xv[PER4];
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < PER4; ++e) {
    const int c = g0 + threadIdx.x + e * blockDim.x;
    float4 v = c < g1 ? load4(xr + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
    if (n_partials > 0 && c < g1) {
      for (int p0 = 0; p0 < n_partials; p0 += 8) {  // eight slices in flight, added in slice order
        float4 part[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
          part[u] = p0 + u < n_partials ? load4(partials + (p0 + u) * partial_stride + src + 4 * c)
                                        : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (p0 + u < n_partials) v.x += part[u].x, v.y += part[u].y, v.z += part[u].z, v.w += part[u].w;
      }
      if (rows == nullptr) store4(xr + 4 * c, v);
    }
    xv[e] = v;
    ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
  }
  const float mine = block_sum(ss, scratch);
  if (threadIdx.x < ranks) {  // thread k tells rank k
    uint32_t remote;
    const uint32_t local = static_cast<uint32_t>(__cvta_generic_to_shared(&shares[rank]));
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(threadIdx.x));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(mine) : "memory");
  }
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  float total = 0.f;
  for (int k = 0; k < ranks; ++k) total += shares[k];
  const float inv = 1.0f / sqrtf(total / static_cast<float>(hidden) + eps);
#pragma unroll
  for (int e = 0; e < PER4; ++e) {
    const int c = g0 + threadIdx.x + e * blockDim.x;
    if (c < g1)
      store4(yr + 4 * c, make_float4((xv[e].x * inv) * wv[e].x, (xv[e].y * inv) * wv[e].y,
                                     (xv[e].z * inv) * wv[e].z, (xv[e].w * inv) * wv[e].w));
  }
}

int g_lrm_norm_ranks = 0;  // 0: the rule in launch_norm; 1: never a cluster; 2, 4, 8: always that many (tuning)

template <typename W, typename O, int PER4>
static int launch_norm_cluster(float* x, const W* w, O* out, const int* rows, const float* partials,
                               int n_partials, size_t partial_stride, int n_rows, int hidden, float eps,
                               int ranks, int threads, cudaStream_t stream) {
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(n_rows * ranks);
  config.blockDim = dim3(threads);
  config.stream = stream;
  cudaLaunchAttribute attributes[2];
  attributes[0].id = cudaLaunchAttributeClusterDimension;
  attributes[0].val.clusterDim.x = ranks;
  attributes[0].val.clusterDim.y = 1;
  attributes[0].val.clusterDim.z = 1;
  attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attributes[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attributes;
  config.numAttrs = g_lrm_pdl ? 2 : 1;
  return static_cast<int>(cudaLaunchKernelEx(&config, rms_norm_cluster_kernel<W, O, PER4>, x, w, out, rows, partials,
                                             n_partials, partial_stride, hidden, eps, ranks));
}

template <typename W, typename O>
static int launch_norm(float* x, const void* w, void* out, const int* rows, const float* partials,
                        int n_partials, size_t partial_stride, int n_rows, int hidden, float eps,
                        cudaStream_t stream) {
  auto aligned = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  if (hidden % 4 == 0 && aligned(x) && aligned(w) && aligned(out) && aligned(partials)) {
    const int groups = hidden / 4;
    // Few rows of 40 KB or more to read each (the row and the slices to fold), bfloat16 out: a cluster
    // of eight CTAs per row (see the kernel). Whole decode steps, one CTA per row against clusters
    // of 8: 3B sizes at batch 16 2.98 -> 2.86 ms, 8B at batch 8 4.56 -> 4.48, 1B at batch 64 2.10 ->
    // 2.08; rows of 8-24 KB (1B at batch 8) lose 2 % to the cluster's barrier and stay as they were.
    int ranks = g_lrm_norm_ranks;
    if (ranks == 0)
      ranks = sizeof(O) == 2 && n_rows <= 74 && static_cast<long long>(n_partials + 1) * hidden >= 10240 ? 8 : 1;
    if (ranks > 1 && sizeof(O) == 2 && groups >= 32 * ranks) {
      const int per_cta = (groups + ranks - 1) / ranks;
      const int cthreads = per_cta >= 256 ? 256 : 128;
      const int cper4 = (per_cta + cthreads - 1) / cthreads;
#define LRM_NORM_CLUSTER(P4)                                                                                  \
  return launch_norm_cluster<W, O, P4>(x, static_cast<const W*>(w), static_cast<O*>(out), rows, partials,     \
                                       n_partials, partial_stride, n_rows, hidden, eps, ranks, cthreads, stream)
      if (cper4 <= 1) LRM_NORM_CLUSTER(1);
      if (cper4 <= 2) LRM_NORM_CLUSTER(2);
      if (cper4 <= 4) LRM_NORM_CLUSTER(4);
#undef LRM_NORM_CLUSTER
    }
    // up to eight groups of four per thread: 256 threads reach rows of 8,192 elements (a block of
    // 1,024 threads per row was measured at a third of the memory rate at 4,096 elements)
    const int vthreads = groups > 2048 ? 1024 : (groups >= 512 ? 256 : (groups >= 64 ? 128 : 32));
    const int per4 = (groups + vthreads - 1) / vthreads;
#define LRM_NORM_VEC(P4)                                                                               \
  return static_cast<int>(lrm_launch(rms_norm_vec_kernel<W, O, P4>, n_rows, vthreads, 0, stream, x,   \
                                     static_cast<const W*>(w), static_cast<O*>(out), rows, partials,  \
                                     n_partials, partial_stride, hidden, eps))
    if (per4 <= 2) LRM_NORM_VEC(2);
    if (per4 <= 8) LRM_NORM_VEC(8);
#undef LRM_NORM_VEC
  }
  // up to 8 elements per thread for rows up to 8192 long, 32 beyond
  int threads = hidden >= 8192 ? 1024 : (hidden > 2048 ? 1024 : (hidden >= 1024 ? 256 : (hidden >= 256 ? 128 : 32)));
#define LRM_NORM_PER(PER)                                                                         \
  return static_cast<int>(lrm_launch(rms_norm_kernel<W, O, PER>, n_rows, threads, 0, stream, x,  \
                                     static_cast<const W*>(w), static_cast<O*>(out), rows,       \
                                     partials, n_partials, partial_stride, hidden, eps))
  const int per = (hidden + threads - 1) / threads;
  if (per <= 8) LRM_NORM_PER(8);
  if (per <= 32) LRM_NORM_PER(32);
  return LRM_UNSUPPORTED;  // rows longer than 32768 elements
#undef LRM_NORM_PER
}

LRM_API int lrm_rms_norm(float* x, const void* w, int w_dtype, void* out, int out_dtype,
                         const int* rows, const float* partials, int n_partials,
                         long long partial_stride, int n_rows, int hidden, float eps,
                         cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (hidden <= 0 || !(eps > 0.f)) return LRM_BAD_ARGUMENT;
  const size_t ps = static_cast<size_t>(partial_stride);
#define LRM_NORM(WT, OT) launch_norm<WT, OT>(x, w, out, rows, partials, n_partials, ps, n_rows, hidden, eps, stream)
  if (w_dtype == LRM_F32 && out_dtype == LRM_F32) return LRM_NORM(float, float);
  if (w_dtype == LRM_F32 && out_dtype == LRM_BF16) return LRM_NORM(float, __nv_bfloat16);
  if (w_dtype == LRM_BF16 && out_dtype == LRM_F32) return LRM_NORM(__nv_bfloat16, float);
  if (w_dtype == LRM_BF16 && out_dtype == LRM_BF16) return LRM_NORM(__nv_bfloat16, __nv_bfloat16);
  return LRM_BAD_ARGUMENT;
#undef LRM_NORM
}

// Tuning and tests: 0 leaves the choice between one CTA and a cluster per row to the kernel's rule,
// 1 never uses a cluster, 2, 4 or 8 always use one of that size (where the output is bfloat16).
LRM_API void lrm_set_norm_ranks(int ranks) { g_lrm_norm_ranks = ranks; }
