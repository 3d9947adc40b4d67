// Causal grouped-query flash attention for prompts on the 5th-generation tensor cores.
//
// One CTA = 128 queries of one head of one sequence; keys and values arrive in tiles of 128
// through TMA (cp.async.bulk.tensor, 128-byte swizzle, two stages). Per key tile:
//   S = Q K^T      tcgen05.mma, M 128 x N 128, K = head size, into tensor memory
//   softmax        eight warps, two threads per query row (each takes 64 of the tile's keys; the
//                  two exchange the row's maximum through a spare column of tensor memory):
//                  tcgen05.ld of the half row, scale, causal and window mask, running max and mass
//                  in float32 (log2 domain), P = 2^(s - m) rounded to bfloat16 and written to
//                  shared memory in the operand layout
//   PV = P V       tcgen05.mma, M 128 x N = head size, K 128, V read as an MN-major operand
//                  exactly as TMA laid it down ([key][d] rows of 128 bytes)
//   O = O a + PV   in registers, half of the head's columns per thread (a = 2^(m_old - m_new)),
//                  tcgen05.ld of PV
// The next tile's S is issued as soon as the probabilities of the current one are written, so
// it runs under the current tile's PV and rescale. Head sizes 64 and 128.
// Rows and keys outside a sequence are zero-filled by TMA or belong to a neighbouring sequence
// of the packed batch; the causal mask hides such keys and such rows are never stored.
// Every mbarrier wait is bounded; a wait that gives up records a code in `status`, and the CTA
// winds down and frees its tensor memory. No cluster multicast.
// (Reference: crates/metal-backend/src/shaders/attention.metal:28-57, the streaming softmax.)
#include "umma.cuh"

namespace {

constexpr int BQ = 128, BKV = 128, UMMA_K = 16;

__device__ __forceinline__ void pair_barrier(int id) {  // the two warps that share a row quadrant
  asm volatile("bar.sync %0, 64;" ::"r"(id) : "memory");
}

constexpr int kSoftmaxWarps = 8;   // two per 32 query rows: each takes half of a tile's keys
constexpr int kThreadsPerCta = (kSoftmaxWarps + 1) * 32;

enum : int { kStuckQ = 11, kStuckKV = 12, kStuckScores = 13, kStuckProbabilities = 14, kStuckValues = 15,
             kStuckStage = 16, kMisaligned = 17 };

// Shared memory (1024-byte aligned): Q [128][D] | 2 stages of (K [128][D] | V [128][D]) |
// P [2 blocks of 64 keys][128 rows][64] | barriers. A [128][D] tile with D = 128 is two
// [128][64] blocks of 16 KB one after the other (a swizzle row is 128 bytes = 64 elements).
template <int D>
__global__ __launch_bounds__(kThreadsPerCta, D == 64 ? 2 : 1) void attention_prefill_umma_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out,
    const int* __restrict__ cu_seqlens, int q_heads, int kv_heads, float scale_log2, int window,
    int* __restrict__ status) {
  constexpr uint32_t TILE = BQ * D * 2;       // bytes of one [128][D] tile
  constexpr uint32_t BLOCK = BQ * 64 * 2;     // bytes of one [128][64] block
  constexpr int DB = D / 64;                  // 64-column blocks per tile
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // The kernel has no static shared memory, so the dynamic block starts 1024-byte aligned, which
  // the swizzled tiles need; should that ever not hold, give up rather than compute nonsense.
  if ((smem_u32(smem_raw) & 1023u) != 0) {
    if (threadIdx.x == 0 && status != nullptr) atomicCAS(status, 0, kMisaligned);
    return;
  }
  unsigned char* q_tile = smem_raw;
  unsigned char* kv_tiles = q_tile + TILE;                 // stage s: K at s * 2 * TILE, V right after
  unsigned char* p_tile = kv_tiles + 4 * TILE;             // [2][128][64] bf16
  uint64_t* bars = reinterpret_cast<uint64_t*>(p_tile + 2 * BLOCK);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;     // [2]
  uint64_t* kv_free = bars + 3;     // [2]
  uint64_t* s_full = bars + 5;
  uint64_t* p_ready = bars + 6;
  uint64_t* pv_full = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* bail = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* pair_fail = bail + 1;  // [2 parities][4 pairs of warps]

  // CTAs are handed out in the order x, y, z: all heads and sequences of the last query tile
  // (the longest rows of work under the causal mask) first, the first query tile last, so the
  // tail of the grid is made of short CTAs.
  const int qt = gridDim.z - 1 - blockIdx.z;
  const int h = blockIdx.x, b = blockIdx.y;
  const int start = cu_seqlens[b], len = cu_seqlens[b + 1] - start;
  const int q0 = qt * BQ;
  if (q0 >= len) return;
  const int kh = h / (q_heads / kv_heads);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kt_first = window > 0 ? max(0, q0 - window + 1) / BKV : 0;
  const int n_tiles = qt - kt_first + 1;  // key tiles up to the diagonal one

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(kv_full + s, 1);
      mbar_init(kv_free + s, 1);
    }
    mbar_init(s_full, 1);
    mbar_init(p_ready, kSoftmaxWarps);
    mbar_init(pv_full, 1);
    *bail = 0;
    for (int i = 0; i < 8; ++i) pair_fail[i] = 0;
    mbar_fence_init();
  }
  constexpr uint32_t kTmemColumns = D == 64 ? 256u : 512u;  // scores 128 | weighted values D | 2 to exchange
  if (warp == kSoftmaxWarps) {
    tmem_alloc(tmem_slot, kTmemColumns);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_s = *tmem_slot, tmem_pv = tmem_s + 128, tmem_x = tmem_pv + D;
  // Barriers and tensor memory were set up while the kernel that produces q, k and v may still
  // have been running (sequence bounds are the step's own input); its results are read from here on.
  // (Letting the output projection be scheduled before this kernel's CTAs exit was measured too:
  // a 2,048-token prompt took 4.85 ms instead of 4.81.)
  pdl_wait();

  if (warp == kSoftmaxWarps) {
    if (lane == 0) {
      // ---- one thread loads tiles and issues the MMAs
      auto load_kv = [&](int j) {
        const int s = j & 1, row = start + (kt_first + j) * BKV;
        unsigned char* kdst = kv_tiles + s * 2 * TILE;
        mbar_expect_tx(kv_full + s, 2 * TILE);
#pragma unroll
        for (int db = 0; db < DB; ++db) {
          tma_load_2d(kdst + db * BLOCK, &map_k, kv_full + s, kh * D + db * 64, row);
          tma_load_2d(kdst + TILE + db * BLOCK, &map_v, kv_full + s, kh * D + db * 64, row);
        }
      };
      mbar_expect_tx(q_full, TILE);
#pragma unroll
      for (int db = 0; db < DB; ++db) tma_load_2d(q_tile + db * BLOCK, &map_q, q_full, h * D + db * 64, start + q0);
      load_kv(0);
      if (n_tiles > 1) load_kv(1);

      // instruction descriptors: D float32, A and B bfloat16, M 128; S: N 128, both K-major;
      // PV: N = head size, B (V) MN-major (bit 16)
      constexpr uint32_t common = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(BQ >> 4) << 24);
      constexpr uint32_t idesc_s = common | (static_cast<uint32_t>(BKV >> 3) << 17);
      constexpr uint32_t idesc_pv = common | (static_cast<uint32_t>(D >> 3) << 17) | (1u << 16);
      auto issue_scores = [&](int j) {
        const uint32_t qa = smem_u32(q_tile), ka = smem_u32(kv_tiles + (j & 1) * 2 * TILE);
#pragma unroll
        for (int k = 0; k < D / UMMA_K; ++k) {
          const uint32_t off = (k / 4) * BLOCK + (k % 4) * UMMA_K * 2;  // 64-column block, then 32 bytes per step
          umma_bf16(tmem_s, smem_desc(qa + off, 16), smem_desc(ka + off, 16), idesc_s, k > 0 ? 1u : 0u);
        }
        umma_commit(s_full);
      };
      bool ok = mbar_wait(q_full, 0, status, kStuckQ) && mbar_wait(kv_full, 0, status, kStuckKV);
      if (ok) {
        tc_fence_after();
        issue_scores(0);
      }
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j & 1;
        ok = mbar_wait(p_ready, j & 1, status, kStuckProbabilities);
        if (!ok) break;
        tc_fence_after();
        const uint32_t pa = smem_u32(p_tile), va = smem_u32(kv_tiles + s * 2 * TILE + TILE);
#pragma unroll
        for (int k = 0; k < BKV / UMMA_K; ++k) {
          // P: K-major, block of 64 keys then 32 bytes per step; V: MN-major, 16 keys = 2048 bytes
          // per step, 64-column blocks 16 KB apart
          umma_bf16(tmem_pv, smem_desc(pa + (k / 4) * BLOCK + (k % 4) * UMMA_K * 2, 16),
                    smem_desc(va + k * UMMA_K * 128, BLOCK), idesc_pv, k > 0 ? 1u : 0u);
        }
        umma_commit(pv_full);
        umma_commit(kv_free + s);
        if (j + 1 < n_tiles) {
          ok = mbar_wait(kv_full + ((j + 1) & 1), ((j + 1) >> 1) & 1, status, kStuckKV);
          if (!ok) break;
          tc_fence_after();
          issue_scores(j + 1);
        }
        if (j + 2 < n_tiles) {
          ok = mbar_wait(kv_free + s, (j >> 1) & 1, status, kStuckStage);
          if (!ok) break;
          load_kv(j + 2);
        }
      }
      if (!ok) *bail = 1;
    }
  } else {
    // ---- softmax and output: two threads per query row. Warps w and w + 4 own the same 32 rows
    // (TMEM lanes): warp w < 4 takes the first 64 keys of every tile and the first half of the
    // head's columns, warp w + 4 the rest. The pair exchanges the row's maximum (and at the end
    // its mass) through two spare TMEM columns and meets at a named barrier of its own.
    const int quad = warp & 3, half = warp >> 2;
    const int row = q0 + quad * 32 + lane;       // position in the sequence
    constexpr int DH = D / 2;                    // output columns per thread
    float o[DH];
#pragma unroll
    for (int d = 0; d < DH; ++d) o[d] = 0.f;
    float m = -INFINITY, l = 0.f;
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      // A wait that gave up is told to the partner warp before the pair's barrier, in a flag that
      // only this pair writes and only for this parity, so both warps leave the loop together.
      if (!(!*bail && mbar_wait(s_full, j & 1, status, kStuckScores))) {
        pair_fail[(j & 1) * 4 + quad] = 1;
        *bail = 1;
      }
      tc_fence_after();
      const int key0 = (kt_first + j) * BKV;
      const bool edge = key0 + BKV - 1 > q0 || (window > 0 && key0 <= q0 + BQ - 1 - window);
      // pass 1: the maximum of this thread's half of the row (only tiles on the diagonal or the
      // window's edge need the mask)
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t r[32];
        tmem_load32(tmem_s + lane_base + half * 64 + c * 32, r);
        if (edge) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int key = key0 + half * 64 + c * 32 + i;
            if (key <= row && (window <= 0 || key > row - window)) mx = fmaxf(mx, __uint_as_float(r[i]));
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(r[i]));
        }
      }
      tmem_store1(tmem_x + lane_base + half, __float_as_uint(mx));
      tc_fence_before();
      pair_barrier(1 + quad);
      tc_fence_after();
      if (pair_fail[(j & 1) * 4 + quad]) {
        ok = false;
        break;
      }
      mx = fmaxf(mx, __uint_as_float(tmem_load1(tmem_x + lane_base + (half ^ 1))));
      const float m_new = fmaxf(m, mx * scale_log2);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = fast_exp2(m - m_use);
      // pass 2: probabilities, rounded to bfloat16, into the operand tile: keys 64 half .. + 63 are
      // block `half` (row = this thread's; 16-byte chunk c of a 128-byte row goes to chunk c ^ (row & 7))
      float sum = 0.f;
      unsigned char* prow = p_tile + half * BLOCK + (quad * 32 + lane) * 128;
      const int swz = (quad * 32 + lane) & 7;
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t r[32];
        tmem_load32(tmem_s + lane_base + half * 64 + c * 32, r);
        uint32_t packed[16];
        if (edge) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const int key = key0 + half * 64 + c * 32 + i;
            const bool v0 = key <= row && (window <= 0 || key > row - window);
            const bool v1 = key + 1 <= row && (window <= 0 || key + 1 > row - window);
            const float p0 = v0 ? fast_exp2(fmaf(__uint_as_float(r[i]), scale_log2, -m_use)) : 0.f;
            const float p1 = v1 ? fast_exp2(fmaf(__uint_as_float(r[i + 1]), scale_log2, -m_use)) : 0.f;
            sum += p0 + p1;
            packed[i >> 1] = pack_bf16(p0, p1);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float p0 = fast_exp2(fmaf(__uint_as_float(r[i]), scale_log2, -m_use));
            const float p1 = fast_exp2(fmaf(__uint_as_float(r[i + 1]), scale_log2, -m_use));
            sum += p0 + p1;
            packed[i >> 1] = pack_bf16(p0, p1);
          }
        }
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {  // 32 keys = 4 chunks of 16 bytes
          const int chunk = c * 4 + q4;
          *reinterpret_cast<uint4*>(prow + ((chunk ^ swz) << 4)) =
              make_uint4(packed[4 * q4], packed[4 * q4 + 1], packed[4 * q4 + 2], packed[4 * q4 + 3]);
        }
      }
      l = l * alpha + sum;
      m = m_new;
      tc_fence_before();
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> tensor core reads
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready);
      // rescale while the tensor core multiplies
#pragma unroll
      for (int d = 0; d < DH; ++d) o[d] *= alpha;
      if (mbar_wait(pv_full, j & 1, status, kStuckValues)) {
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < DH / 32; ++c) {
          uint32_t r[32];
          tmem_load32(tmem_pv + lane_base + half * DH + c * 32, r);
#pragma unroll
          for (int i = 0; i < 32; ++i) o[c * 32 + i] += __uint_as_float(r[i]);
        }
        tc_fence_before();
      } else {  // seen by both warps of the pair after the next barrier
        pair_fail[((j + 1) & 1) * 4 + quad] = 1;
        *bail = 1;
      }
    }
    // the pair adds up the row's mass; both warps are here for the same reason
    if (ok) {
      tmem_store1(tmem_x + lane_base + half, __float_as_uint(l));
      tc_fence_before();
      pair_barrier(1 + quad);
      tc_fence_after();
      ok = !pair_fail[(n_tiles & 1) * 4 + quad];
      l += __uint_as_float(tmem_load1(tmem_x + lane_base + (half ^ 1)));
    }
    if (!ok) *bail = 1;
    if (ok && row < len) {
      const float inv = 1.0f / l;
      __nv_bfloat16* dst = out + (static_cast<size_t>(start + row) * q_heads + h) * D + half * DH;
#pragma unroll
      for (int d = 0; d < DH; d += 8)
        *reinterpret_cast<uint4*>(dst + d) =
            make_uint4(pack_bf16(o[d] * inv, o[d + 1] * inv), pack_bf16(o[d + 2] * inv, o[d + 3] * inv),
                       pack_bf16(o[d + 4] * inv, o[d + 5] * inv), pack_bf16(o[d + 6] * inv, o[d + 7] * inv));
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kSoftmaxWarps)
    tmem_dealloc(tmem_s, kTmemColumns);
}

template <int D>
int launch(const void* q, const void* k, const void* v, void* out, const int* cu_seqlens, int tokens,
           int seqs, int max_seq_len, int q_heads, int kv_heads, float scale, int window, int* status,
           cudaStream_t stream) {
  CUtensorMap map_q, map_k, map_v;
  if (!make_map_bf16(&map_q, q, tokens, static_cast<long long>(q_heads) * D, BQ) ||
      !make_map_bf16(&map_k, k, tokens, static_cast<long long>(kv_heads) * D, BKV) ||
      !make_map_bf16(&map_v, v, tokens, static_cast<long long>(kv_heads) * D, BKV))
    return LRM_UNSUPPORTED;
  constexpr int smem = 5 * BQ * D * 2 + 2 * BQ * 64 * 2 + 256;
  auto kernel = attention_prefill_umma_kernel<D>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (seqs > 65535 || (max_seq_len + BQ - 1) / BQ > 65535) return LRM_UNSUPPORTED;
  const dim3 grid(q_heads, seqs, (max_seq_len + BQ - 1) / BQ);
  LRM_LAUNCH(kernel, grid, dim3(kThreadsPerCta), smem, stream, map_q, map_k, map_v, static_cast<__nv_bfloat16*>(out),
             cu_seqlens, q_heads, kv_heads, scale * 1.4426950408889634f, window, status);
  return 0;
}

}  // namespace

LRM_API int lrm_attention_prefill_umma_supports(int head_dim) {
  return (head_dim == 64 || head_dim == 128) && encode_tiled() != nullptr ? 1 : 0;
}

// q [tokens, q_heads, d], k, v [tokens, kv_heads, d] packed bfloat16, 16-byte aligned; `status` as
// in lrm_gemm_bf16_umma.
LRM_API int lrm_attention_prefill_umma(const void* q, const void* k, const void* v, void* out,
                                       const int* cu_seqlens, int tokens, int seqs, int max_seq_len,
                                       int q_heads, int kv_heads, int d, float scale, int window,
                                       int* status, cudaStream_t stream) {
  if (seqs <= 0 || max_seq_len <= 0 || tokens <= 0) return 0;
  if (q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads != 0 || status == nullptr) return LRM_BAD_ARGUMENT;
  if (q_heads > 65535 || seqs > 65535) return LRM_UNSUPPORTED;
  if (reinterpret_cast<uintptr_t>(q) % 16 || reinterpret_cast<uintptr_t>(k) % 16 ||
      reinterpret_cast<uintptr_t>(v) % 16 || reinterpret_cast<uintptr_t>(out) % 16)
    return LRM_UNSUPPORTED;
  if (d == 64)
    return launch<64>(q, k, v, out, cu_seqlens, tokens, seqs, max_seq_len, q_heads, kv_heads, scale, window,
                      status, stream);
  if (d == 128)
    return launch<128>(q, k, v, out, cu_seqlens, tokens, seqs, max_seq_len, q_heads, kv_heads, scale, window,
                       status, stream);
  return LRM_UNSUPPORTED;
}
