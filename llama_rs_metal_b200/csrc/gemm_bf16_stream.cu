// Weight-streaming bfloat16 product for few rows (decode): Y[M,N] = X[M,K] . W[N,K]^T, M <= 64.
//
// Every weight byte is read from HBM exactly once, straight into registers
// with 16-byte loads, and fed to mma.sync m16n8k16 with the weights as the
// 16-row operand and the M activation rows as 8-wide column tiles. A thread's
// 16-byte load holds 8 consecutive k of one weight row; the two halves serve
// two consecutive MMAs. Within an MMA the hardware's k index is just a label,
// so the activation fragment is loaded with the same address pattern and the
// products pair up correctly without any shuffle or shared-memory staging.
//
// A CTA owns 16 weight rows; its warps split K into contiguous ranges, streamed in 64- or
// 128-wide chunks (so many loads are in flight per SM), and their partial sums are added in
// warp order through shared memory (no atomics: the result is deterministic).
//
// For a narrow product (few 16-row tiles) that is to be added to the residual stream,
// blockIdx.y may cut K into slices handled by different CTAs, so that every SM still streams.
// Slice s then stores its float32 partial product at out[s] of an [slices, M, N] tensor
// (epilogue 4); whoever reads the residual stream next adds the slices in slice order (the
// norm kernel does it in its own pass). No atomics: the result does not depend on which CTA
// finishes first.
//
// Epilogues: 0 store bf16, 1 store f32, 2 add into f32 in place, 3 SiLU gate
// (rows alternate in blocks of 8 gate / 8 up rows, so a 16-row tile holds 8
// gated pairs; out is [M, N/2] bf16), 4 store f32 partials per K slice, 5 token choice: the
// product is a head's logits and only the chosen token is wanted, so every CTA finds, per
// activation row, the best (score, id) of its 16 vocabulary rows (score = logit for the greedy
// choice, logit / T + Gumbel noise for temperature sampling, as csrc/sampling.cu) and offers it
// to the row's running best with one 64-bit atomic maximum; the logits themselves are never
// written. A maximum does not depend on the order of the offers, so the choice is the same
// every time. lrm_gemm_bf16_stream_pick turns the winners into ids right after (reference: the
// head product and the GPU argmax go out in one submission,
// crates/model-runtime/src/execute.rs:238-247).
// (Reference role: the gemv_* family, crates/metal-backend/src/shaders/matrix.metal:10-37.)
#include "common.cuh"
#include "pick.cuh"

namespace {

// k values a warp handles per iteration: 64 for up to 16 activation rows (fewer registers, so
// more warps per SM), 128 beyond
template <int NT> struct Chunk { static constexpr int kK = NT <= 2 ? 64 : 128; };

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_stream(const void* p) {  // read once: do not keep in L1
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ldg_keep(const void* p) {  // activations: reused by every CTA
  return __ldg(reinterpret_cast<const uint4*>(p));
}

__device__ __forceinline__ float silu_f32(float g) { return g / (1.0f + expf(-g)); }

// What epilogue 5 needs beyond the product's own arguments.
struct PickArgs {
  unsigned long long* best;  // [M] running best per row as pick_key(score, id); 0 before the launch
  int* bad;                  // [M] set when a row held a non-finite logit; 0 before the launch
  const long long* keys;     // [M] per-row stream of the Gumbel noise, or nullptr for the greedy choice
  float inv_temperature;     // scores are logit * this + noise (1 for greedy)
  unsigned long long seed;
};

// MINB: CTAs per SM the register budget must allow (a single wave for the usual sizes).
template <int NT, int WARPS, int MINB>
__global__ __launch_bounds__(WARPS * 32, MINB) void gemm_bf16_stream_kernel(
    const __nv_bfloat16* __restrict__ X, const __nv_bfloat16* __restrict__ W, void* __restrict__ out,
    int M, int N, int K_total, int mode, int k_per_split, PickArgs pick) {
  extern __shared__ float red[];  // [WARPS][NT][32 lanes][4]
  pdl_trigger();  // the next kernel may be scheduled at once (its CTAs fetch their first weights while
                  // this kernel streams); it waits for this one where it must
  constexpr int kChunk = Chunk<NT>::kK, kSub = kChunk / 32;  // kSub: 16-byte pieces per thread and row
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * 16;
  const int k_lo = blockIdx.y * k_per_split;              // this CTA's slice of K: [k_lo, K)
  const int K = min(K_total, k_lo + k_per_split);
  // epilogue 4: this slice's partial product goes to its own [M, N] plane of `out`
  float* plane = mode == 4 ? static_cast<float*>(out) + static_cast<size_t>(blockIdx.y) * M * N : nullptr;
  const int row_a = n0 + g, row_b = n0 + g + 8;
  const bool ok_a = row_a < N, ok_b = row_b < N;
  const __nv_bfloat16* wa = W + static_cast<size_t>(ok_a ? row_a : 0) * K_total;
  const __nv_bfloat16* wb = W + static_cast<size_t>(ok_b ? row_b : 0) * K_total;
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;

  // Each warp streams one contiguous range of k (so that what it has in flight is adjacent in
  // memory): [k0, k_end), a whole number of chunks except at the end of the slice.
  const int per_warp = ((K - k_lo + WARPS - 1) / WARPS + kChunk - 1) / kChunk * kChunk;
  int k0 = k_lo + warp * per_warp;
  const int k_end = min(K, k0 + per_warp);
  auto load_w = [&](int k0, uint4 (&a)[kSub], uint4 (&b)[kSub]) {
#pragma unroll
    for (int s = 0; s < kSub; ++s) {
      const int k = k0 + 32 * s + 8 * t;
      const bool in = k < k_end;  // a multiple of 8: a 16-byte piece is inside or outside
      a[s] = in && ok_a ? ldg_stream(wa + k) : zero;
      b[s] = in && ok_b ? ldg_stream(wb + k) : zero;
    }
  };

  // Weights do not depend on the kernel before this one: start streaming them, then wait
  // for the predecessor (which produced X and may still be writing `out`). Each warp keeps the
  // next chunk in flight while it multiplies the current one.
  uint4 cur_a[kSub], cur_b[kSub], nxt_a[kSub], nxt_b[kSub];
  if (k0 < k_end) load_w(k0, cur_a, cur_b);
  if (k0 + kChunk < k_end) load_w(k0 + kChunk, nxt_a, nxt_b);
  pdl_wait();
  // mode 2 adds into `out`: fetch the old values now so their latency hides behind the stream
  float old[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
  if (mode == 2 && threadIdx.x < NT * 32) {
    const int j = threadIdx.x >> 5, gg = (threadIdx.x & 31) >> 2, tt = threadIdx.x & 3;
#pragma unroll
    for (int e = 0; e < 2; ++e)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int m = 8 * j + 2 * tt + e, n = n0 + gg + 8 * half;
        if (m < M && n < N) old[e][half] = static_cast<const float*>(out)[static_cast<size_t>(m) * N + n];
      }
  }
  bool first = true;
  while (k0 < k_end) {
    const int k_next = k0 + kChunk;
    if (!first && k_next < k_end) load_w(k_next, nxt_a, nxt_b);  // the first pair was fetched before the wait
    first = false;
#pragma unroll
    for (int s = 0; s < kSub; ++s) {
      const int k = k0 + 32 * s + 8 * t;
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        const int m = 8 * j + g;
        const uint4 x = (m < M && k < k_end) ? ldg_keep(X + static_cast<size_t>(m) * K_total + k) : zero;
        mma16816(acc[j], cur_a[s].x, cur_b[s].x, cur_a[s].y, cur_b[s].y, x.x, x.y);
        mma16816(acc[j], cur_a[s].z, cur_b[s].z, cur_a[s].w, cur_b[s].w, x.z, x.w);
      }
    }
    k0 = k_next;
#pragma unroll
    for (int s = 0; s < kSub; ++s) {
      cur_a[s] = nxt_a[s];
      cur_b[s] = nxt_b[s];
    }
  }

  // add the warps' partial sums in warp order
#pragma unroll
  for (int j = 0; j < NT; ++j)
    *reinterpret_cast<float4*>(red + ((static_cast<size_t>(warp) * NT + j) * 32 + lane) * 4) =
        make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
  __syncthreads();
  for (int item = threadIdx.x; item < NT * 32; item += WARPS * 32) {
    const int j = item >> 5, ln = item & 31, gg = ln >> 2, tt = ln & 3;
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      const float4 v = *reinterpret_cast<const float4*>(red + ((static_cast<size_t>(w) * NT + j) * 32 + ln) * 4);
      sum.x += v.x;
      sum.y += v.y;
      sum.z += v.z;
      sum.w += v.w;
    }
    // sum.x/.y: weight row n0+gg, batch rows 8j+2tt, +1;  sum.z/.w: weight row n0+gg+8
    const int m0 = 8 * j + 2 * tt;
    const float vals[2][2] = {{sum.x, sum.z}, {sum.y, sum.w}};  // [batch row offset][weight row half]
    if (mode == 5) {
      // This warp holds tile j's 8 activation rows x 16 vocabulary rows: a lane has rows m0, m0 + 1
      // and vocabulary ids n0 + gg, n0 + gg + 8. The best of a row's 16 is found over the lanes
      // that share tt (xor 4, 8, 16); ties go to the lower id, so the result does not depend on
      // how the vocabulary is cut into tiles.
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int m = m0 + e;
        Best best{-INFINITY, -1};
        bool bad = false;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int n = n0 + gg + 8 * half;
          if (n >= N || m >= M) continue;
          float v = vals[e][half];
          bad |= !isfinite(v);
          if (pick.keys != nullptr)
            v = fmaf(v, pick.inv_temperature,
                     gumbel_noise(pick.seed, static_cast<uint64_t>(pick.keys[m]), static_cast<uint32_t>(n)));
          best = better(best, Best{v, n});
        }
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
          Best other{__shfl_xor_sync(0xffffffffu, best.value, o), __shfl_xor_sync(0xffffffffu, best.id, o)};
          best = better(best, other);
          bad |= __shfl_xor_sync(0xffffffffu, static_cast<int>(bad), o) != 0;
        }
        if (gg == 0 && m < M) {
          if (best.id >= 0) atomicMax(pick.best + m, pick_key(best.value, best.id));
          if (bad) atomicOr(pick.bad + m, 1);
        }
      }
      continue;
    }
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int m = m0 + e;
      if (m >= M) continue;
      if (mode == 3) {
        const int col = (n0 >> 1) + gg;  // gate row n0+gg pairs with up row n0+gg+8
        if (n0 + gg + 8 < N)
          static_cast<__nv_bfloat16*>(out)[static_cast<size_t>(m) * (N >> 1) + col] =
              __float2bfloat16_rn(silu_f32(vals[e][0]) * vals[e][1]);
        continue;
      }
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int n = n0 + gg + 8 * half;
        if (n >= N) continue;
        const size_t o = static_cast<size_t>(m) * N + n;
        const float v = vals[e][half];
        if (mode == 0) static_cast<__nv_bfloat16*>(out)[o] = __float2bfloat16_rn(v);
        else if (mode == 1) static_cast<float*>(out)[o] = v;
        else if (mode == 4) plane[o] = v;
        else static_cast<float*>(out)[o] = (item < WARPS * 32 ? old[e][half] : static_cast<float*>(out)[o]) + v;
      }
    }
  }
}

template <int NT, int WARPS, int MINB>
int launch_variant(const void* X, const void* W, void* out, int M, int N, int K, int mode, int splits,
                   const PickArgs& pick, cudaStream_t stream) {
  constexpr int smem = WARPS * NT * 32 * 4 * static_cast<int>(sizeof(float));
  auto kernel = gemm_bf16_stream_kernel<NT, WARPS, MINB>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  constexpr int kChunk = Chunk<NT>::kK;
  const int k_per_split = ((K + splits - 1) / splits + kChunk - 1) / kChunk * kChunk;
  const dim3 grid((N + 15) / 16, (K + k_per_split - 1) / k_per_split);
  LRM_LAUNCH(kernel, grid, WARPS * 32, smem, stream, static_cast<const __nv_bfloat16*>(X),
             static_cast<const __nv_bfloat16*>(W), out, M, N, K, mode, k_per_split, pick);
  return 0;
}

// Register budgets: 64 per thread for up to 16 activation rows (32 warps resident per SM),
// 128 beyond (the accumulators of 4 or 8 column tiles need them).
template <int NT>
int launch_stream(const void* X, const void* W, void* out, int M, int N, int K, int mode, int warps,
                  int splits, const PickArgs& pick, cudaStream_t stream) {
  constexpr int kWarpsPerSm = NT <= 2 ? 32 : 16;
  if (warps >= 16) return launch_variant<NT, 16, kWarpsPerSm / 16>(X, W, out, M, N, K, mode, splits, pick, stream);
  if (warps >= 8) return launch_variant<NT, 8, kWarpsPerSm / 8>(X, W, out, M, N, K, mode, splits, pick, stream);
  if (warps >= 4) return launch_variant<NT, 4, kWarpsPerSm / 4>(X, W, out, M, N, K, mode, splits, pick, stream);
  if (warps >= 2) return launch_variant<NT, 2, kWarpsPerSm / 2>(X, W, out, M, N, K, mode, splits, pick, stream);
  return launch_variant<NT, 1, kWarpsPerSm>(X, W, out, M, N, K, mode, splits, pick, stream);
}

int launch_rows(const void* X, const void* W, void* out, int M, int N, int K, int mode, int warps, int splits,
                const PickArgs& pick, cudaStream_t stream) {
  // enough warps per CTA that each has at least one chunk
  const int tiles = (N + 15) / 16;
  const int chunks = ((K + splits - 1) / splits + 127) / 128;
  if (warps == 0) {
    warps = 4;
    while (warps < 16 && tiles * splits * warps < 148 * 16 && warps * 2 <= chunks) warps *= 2;
    while (warps > 1 && warps > chunks) warps /= 2;
  }
  if (M <= 8) return launch_stream<1>(X, W, out, M, N, K, mode, warps, splits, pick, stream);
  if (M <= 16) return launch_stream<2>(X, W, out, M, N, K, mode, warps, splits, pick, stream);
  if (M <= 32) return launch_stream<4>(X, W, out, M, N, K, mode, warps, splits, pick, stream);
  return launch_stream<8>(X, W, out, M, N, K, mode, warps < 8 ? warps : 8, splits, pick, stream);
}

}  // namespace

// Shapes this kernel takes: at most 64 rows, K a multiple of 8, 16-byte aligned operands.
LRM_API int lrm_gemm_bf16_stream_supports(int M, int N, int K) {
  return M >= 1 && M <= 64 && N >= 1 && K >= 8 && K % 8 == 0 ? 1 : 0;
}

static int chunk_of(int M) { return M <= 16 ? 64 : 128; }  // Chunk<NT>::kK for this many rows

// How many K slices a product to be added to the residual stream is cut into: `requested`, or with
// 0 the kernel's own rule: slices of at least 4096 until about 28 warps per SM stream weights.
// (Measured over a 16-layer chain of the 1B products at 1-8 rows: the 2048 x 8192 product in two
// slices and the 2048 x 2048 one whole take 495 us, against 540 us with 8 and 2 slices and 568 us
// uncut; every plane costs the norm that adds it a read that only as many SMs share as there are
// rows.) The answer is the number of [M, N] planes epilogue 4 writes.
static int pick_splits(int N, int K, int requested) {
  if (requested > 0) return requested;
  const int tiles = (N + 15) / 16;
  int splits = 1;
  while (splits < 8 && tiles * splits * 8 < 148 * 28 && K / (splits * 2) >= 4096) splits *= 2;
  return splits;
}

LRM_API int lrm_gemm_bf16_stream_slices(int M, int N, int K, int requested) {
  if (M <= 0 || N <= 0 || K <= 0) return 1;
  const int splits = pick_splits(N, K, requested);
  const int chunk = chunk_of(M);
  const int k_per_split = ((K + splits - 1) / splits + chunk - 1) / chunk * chunk;
  return (K + k_per_split - 1) / k_per_split;
}

// `warps` (1, 2, 4, 8, 16) chooses the launch shape, 0 leaves it to the rule below. `splits`: K
// slices, epilogue 4 only (out then holds lrm_gemm_bf16_stream_slices(M, N, K, splits) planes).
LRM_API int lrm_gemm_bf16_stream_shaped(const void* X, const void* W, void* out, int M, int N, int K,
                                        int mode, int warps, int splits, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (!lrm_gemm_bf16_stream_supports(M, N, K)) return LRM_UNSUPPORTED;
  if (mode < 0 || mode > 4 || (mode == 3 && N % 16 != 0)) return LRM_BAD_ARGUMENT;
  if (warps < 0 || warps > 16 || splits < 0 || splits > 64 || (splits > 1 && mode != 4)) return LRM_BAD_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(X) % 16 || reinterpret_cast<uintptr_t>(W) % 16) return LRM_UNSUPPORTED;
  splits = mode == 4 ? pick_splits(N, K, splits) : 1;
  return launch_rows(X, W, out, M, N, K, mode, warps, splits, PickArgs{}, stream);
}

// The head product with the token choice in its epilogue: ids[m] = the chosen vocabulary row for
// activation row m of X [M, K] against W [N, K] (N = vocabulary), never writing the logits.
// keys == nullptr: greedy (largest logit, lowest id on ties). Otherwise a draw from
// softmax(logits / temperature) by Gumbel-max with the noise of lrm_sample_gumbel_rows (same
// seed, keys and hash), so both ways choose the same token from the same logits. A row with a
// non-finite logit gives -1. Scratch: `best` (M 64-bit words) and `bad` (M ints), all zero before
// the call and zero again after it (the second kernel clears what it read), so one allocation
// serves every call that follows on the same stream; calls that overlap on the GPU must not
// share it. Two launches (the product, then the winners' ids).
LRM_API int lrm_gemm_bf16_stream_pick(const void* X, const void* W, int M, int N, int K,
                                      unsigned long long* best, int* bad, int* ids, float temperature,
                                      unsigned long long seed, const long long* keys, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (N <= 0 || !lrm_gemm_bf16_stream_supports(M, N, K)) return LRM_UNSUPPORTED;
  if (best == nullptr || bad == nullptr || ids == nullptr) return LRM_BAD_ARGUMENT;
  if (keys != nullptr && !(temperature > 0.f)) return LRM_BAD_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(X) % 16 || reinterpret_cast<uintptr_t>(W) % 16) return LRM_UNSUPPORTED;
  PickArgs pick{best, bad, keys, keys != nullptr ? 1.0f / temperature : 1.0f, seed};
  const int code = launch_rows(X, W, nullptr, M, N, K, 5, 0, 1, pick, stream);
  if (code != 0) return code;
  return lrm_pick_winners(best, bad, ids, M, stream);
}

LRM_API int lrm_gemm_bf16_stream(const void* X, const void* W, void* out, int M, int N, int K,
                                 int mode, cudaStream_t stream) {
  return lrm_gemm_bf16_stream_shaped(X, W, out, M, N, K, mode, 0, 0, stream);
}
