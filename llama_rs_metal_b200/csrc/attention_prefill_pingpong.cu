// Causal grouped-query flash attention for prompts on the 5th-generation tensor cores, with
// scores, probabilities and output in tensor memory and two query tiles taking turns on each
// SM's tensor core.
//
// One CTA = one or two tiles of 128 queries of one head of one sequence; keys and values arrive
// in tiles of 128 through TMA (cp.async.bulk.tensor, 128-byte swizzle, a ring of stages). For
// query tile i and key tile j:
//   S_i = Q_i K_j^T   tcgen05.mma, M 128 x N 128, K = head size, into tensor memory
//   softmax           four warps per query tile, one thread per query row: tcgen05.ld of the row,
//                     scale, causal and window mask, running maximum and mass in float32 (log2
//                     domain), P = 2^(s - m) rounded to bfloat16 and written back into tensor
//                     memory over the scores it came from (two values per column)
//   O_i += P_i V_j    tcgen05.mma with P read from tensor memory as the A operand and V from
//                     shared memory as an MN-major operand exactly as TMA laid it down; O stays
//                     in tensor memory for the whole row of key tiles
// With two query tiles per CTA (head size 128: 256 queries, one CTA per SM) the issuing thread
// alternates between the tiles (P_0 V, the next S_0, P_1 V, the next S_1), so one tile's softmax
// runs under the other tile's products. With one tile per CTA (head size 64: its tiles leave room
// for two CTAs per SM, in shared and in tensor memory) the two CTAs of an SM take turns the same
// way, and short prompts get twice as many CTAs to spread over the SMs. O is rescaled only when a row's
// maximum has moved by more than 2^8 since the scale O was last brought to (the row's own
// thread multiplies its O row in tensor memory); P is formed against that older maximum
// meanwhile and stays below 2^8, and the division by the mass at the end makes the result
// exact regardless. Tensor memory per query tile: S 128 + O D columns.
//
// Rows and keys outside a sequence are zero-filled by TMA or belong to a neighbouring sequence
// of the packed batch; the causal mask hides such keys and such rows are never stored.
// Every mbarrier wait is bounded; a wait that gives up records a code in `status`, and the CTA
// winds down and frees its tensor memory. No cluster multicast. Head sizes 64 and 128.
// (Reference: crates/metal-backend/src/shaders/attention.metal:28-57, the streaming softmax.)
#include "umma.cuh"

namespace {

constexpr int BQ = 128, UMMA_K = 16;
// warps of a CTA with NQ query tiles: four softmax warps per tile, then the loader, then the issuer
constexpr int threads_per_cta(int nq) { return (4 * nq + 2) * 32; }
constexpr float kRescaleStep = 8.0f;                       // log2: O is rescaled when the maximum moved this far

enum : int { kStuckQ = 21, kStuckKV = 22, kStuckScores = 23, kStuckProbabilities = 24, kStuckOutput = 25,
             kStuckStage = 26, kMisaligned = 27 };

// Key/value stages by head size and keys per tile (BKV): with head size 64, one query tile per CTA
// and tiles of 64 keys, four CTAs fit on an SM (two stages and 128 columns of tensor memory each).
template <int D, int BKV> struct Shape {
  static constexpr int kStages = D == 64 && BKV == 128 ? 3 : 2;
  static constexpr int kCtasPerSm = BKV == 64 && D == 64 ? 4 : 2;
};

// Shared memory (1024-byte aligned): Q [2][128][D] | stages of (K [128][D] | V [128][D]) |
// barriers. A [128][D] tile with D = 128 is two [128][64] blocks of 16 KB one after the other
// (a swizzle row is 128 bytes = 64 elements).
template <int D, int NQ, int BKV>
__global__ __launch_bounds__(threads_per_cta(NQ), NQ == 1 ? Shape<D, BKV>::kCtasPerSm : 1)
void attention_prefill_pingpong_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out,
    const int* __restrict__ cu_seqlens, int q_heads, int kv_heads, float scale_log2, int window,
    int* __restrict__ status) {
  constexpr uint32_t TILE = BQ * D * 2;       // bytes of one [128][D] query tile
  constexpr uint32_t BLOCK = BQ * 64 * 2;     // bytes of one [128][64] block of it
  constexpr uint32_t KV_TILE = BKV * D * 2;   // bytes of one [BKV][D] key or value tile
  constexpr uint32_t KV_BLOCK = BKV * 64 * 2; // bytes of one [BKV][64] block of it
  constexpr int DB = D / 64;                  // 64-column blocks per tile
  constexpr int STAGES = Shape<D, BKV>::kStages;
  static_assert(BKV == 128 || (BKV == 64 && NQ == 1), "tiles of 64 keys go with one query tile per CTA");
  constexpr int kLoaderWarp = 4 * NQ, kIssuerWarp = 4 * NQ + 1;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  if ((smem_u32(smem_raw) & 1023u) != 0) {  // the swizzled tiles need it; give up rather than compute nonsense
    if (threadIdx.x == 0 && status != nullptr) atomicCAS(status, 0, kMisaligned);
    return;
  }
  unsigned char* q_tiles = smem_raw;                        // [NQ] tiles
  unsigned char* kv_tiles = q_tiles + NQ * TILE;            // stage s: K at s * 2 * KV_TILE, V right after
  uint64_t* bars = reinterpret_cast<uint64_t*>(kv_tiles + STAGES * 2 * KV_TILE);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;               // [STAGES]
  uint64_t* kv_free = kv_full + STAGES;       // [STAGES]
  uint64_t* s_full = kv_free + STAGES;        // [2] scores of tile i written
  uint64_t* p_ready = s_full + 2;             // [2] probabilities of tile i written (4 warps arrive)
  uint64_t* o_done = p_ready + 2;             // [2] the last P V of tile i is complete
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_done + 2);
  volatile int* bail = reinterpret_cast<volatile int*>(tmem_slot + 1);

  // CTAs are handed out in the order x, y, z: all heads and sequences of the last pair of query
  // tiles (the longest rows of work under the causal mask) first.
  const int pair = gridDim.z - 1 - blockIdx.z;
  const int h = blockIdx.x, b = blockIdx.y;
  const int start = cu_seqlens[b], len = cu_seqlens[b + 1] - start;
  const int q0 = pair * NQ * BQ;
  if (q0 >= len) return;
  const int kh = h / (q_heads / kv_heads);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kt_first = window > 0 ? max(0, q0 - window + 1) / BKV : 0;
  // key tiles per query tile: up to its diagonal tile; the second tile may not exist
  const int n0 = (q0 + BQ - 1) / BKV - kt_first + 1;
  const int n1 = NQ == 2 && q0 + BQ < len ? n0 + 1 : 0;
  const int n_tiles = max(n0, n1);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(kv_full + s, 1);
      mbar_init(kv_free + s, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(s_full + i, 1);
      mbar_init(p_ready + i, 4);
      mbar_init(o_done + i, 1);
    }
    *bail = 0;
    mbar_fence_init();
  }
  // a power of two that holds NQ (BKV + D) columns
  constexpr uint32_t kTmemColumns = NQ == 2 ? 512 : (BKV + D <= 128 ? 128 : 256);
  if (warp == kIssuerWarp) {
    tmem_alloc(tmem_slot, kTmemColumns);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s[2] = {tmem_base, tmem_base + 128};
  const uint32_t tmem_o[2] = {tmem_base + NQ * BKV, tmem_base + NQ * BKV + D};
  // Barriers and tensor memory were set up while the kernel that produces q, k and v may still
  // have been running (sequence bounds are the step's own input); its results are read from here on.
  pdl_wait();

  if (warp == kLoaderWarp) {
    if (lane == 0) {
      // ---- one thread brings the query tiles once and the key/value tiles through the ring
      mbar_expect_tx(q_full, (n1 > 0 ? 2 : 1) * TILE);
      for (int i = 0; i < (n1 > 0 ? 2 : 1); ++i)
#pragma unroll
        for (int db = 0; db < DB; ++db)
          tma_load_2d(q_tiles + i * TILE + db * BLOCK, &map_q, q_full, h * D + db * 64, start + q0 + i * BQ);
      for (int j = 0; j < n_tiles && !*bail; ++j) {
        const int s = j % STAGES;
        if (j >= STAGES && !mbar_wait(kv_free + s, ((j / STAGES) - 1) & 1, status, kStuckStage)) {
          *bail = 1;
          break;
        }
        const int row = start + (kt_first + j) * BKV;
        unsigned char* kdst = kv_tiles + s * 2 * KV_TILE;
        mbar_expect_tx(kv_full + s, 2 * KV_TILE);
#pragma unroll
        for (int db = 0; db < DB; ++db) {
          tma_load_2d(kdst + db * KV_BLOCK, &map_k, kv_full + s, kh * D + db * 64, row);
          tma_load_2d(kdst + KV_TILE + db * KV_BLOCK, &map_v, kv_full + s, kh * D + db * 64, row);
        }
      }
    }
  } else if (warp == kIssuerWarp) {
    if (lane == 0) {
      // ---- one thread drives the tensor core
      constexpr uint32_t idesc_s = umma_idesc(BQ, BKV);            // both K-major
      constexpr uint32_t idesc_pv = umma_idesc(BQ, D, true);       // V is MN-major
      auto scores = [&](int i, int j) {  // S_i = Q_i K_j^T
        const uint32_t qa = smem_u32(q_tiles + i * TILE), ka = smem_u32(kv_tiles + (j % STAGES) * 2 * KV_TILE);
#pragma unroll
        for (int k = 0; k < D / UMMA_K; ++k) {  // 64-column block, then 32 bytes per step
          const uint32_t step = (k % 4) * UMMA_K * 2;
          umma_bf16(tmem_s[i], smem_desc(qa + (k / 4) * BLOCK + step), smem_desc(ka + (k / 4) * KV_BLOCK + step),
                    idesc_s, k > 0 ? 1u : 0u);
        }
        umma_commit(s_full + i);
      };
      auto weighted = [&](int i, int j) {  // O_i (+)= P_i V_j, P from tensor memory (8 columns per 16 keys)
        const uint32_t va = smem_u32(kv_tiles + (j % STAGES) * 2 * KV_TILE + KV_TILE);
#pragma unroll
        for (int k = 0; k < BKV / UMMA_K; ++k)
          umma_bf16_a_tmem(tmem_o[i], tmem_s[i] + k * (UMMA_K / 2), smem_desc(va + k * UMMA_K * 128, KV_BLOCK),
                           idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
      };
      bool ok = mbar_wait(q_full, 0, status, kStuckQ) && mbar_wait(kv_full, 0, status, kStuckKV);
      if (ok) {
        tc_fence_after();
        scores(0, 0);
        if (n1 > 0) scores(1, 0);
      }
      for (int j = 0; j < n_tiles && ok; ++j) {
        const bool more0 = j + 1 < n0, more1 = j + 1 < n1;
        if (j < n0) {
          ok = mbar_wait(p_ready + 0, j & 1, status, kStuckProbabilities);
          if (!ok) break;
          tc_fence_after();
          weighted(0, j);
          if (j == n0 - 1) umma_commit(o_done + 0);
        }
        if (more0 || more1) {  // the next key tile has to be here for the next scores
          ok = mbar_wait(kv_full + (j + 1) % STAGES, ((j + 1) / STAGES) & 1, status, kStuckKV);
          if (!ok) break;
          tc_fence_after();
        }
        if (more0) scores(0, j + 1);
        if (j < n1) {
          ok = mbar_wait(p_ready + 1, j & 1, status, kStuckProbabilities);
          if (!ok) break;
          tc_fence_after();
          weighted(1, j);
          if (j == n1 - 1) umma_commit(o_done + 1);
        }
        umma_commit(kv_free + j % STAGES);  // every product that reads stage j has been issued
        if (more1) scores(1, j + 1);
      }
      if (!ok) *bail = 1;
    }
  } else {
    // ---- softmax and output: one thread per query row. Warps 0-3 own tile 0, warps 4-7 tile 1;
    // a warp may touch the quarter of the tensor memory's lanes given by its index modulo 4.
    const int i = warp >> 2, quad = warp & 3;
    const int n_mine = i == 0 ? n0 : n1;
    const int row = q0 + i * BQ + quad * 32 + lane;  // position in the sequence
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t my_s = tmem_s[i] + lane_base, my_o = tmem_o[i] + lane_base;
    float m_run = -INFINITY;   // the row's true running maximum (log2 domain)
    float m_ref = -INFINITY;   // the maximum O and the mass are scaled by
    float l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_mine; ++j) {
      if (*bail || !mbar_wait(s_full + i, j & 1, status, kStuckScores)) {
        *bail = 1;
        ok = false;
        break;
      }
      tc_fence_after();
      const int key0 = (kt_first + j) * BKV;
      const int first_row = q0 + i * BQ;
      const bool edge = key0 + BKV - 1 > first_row || (window > 0 && key0 <= first_row + BQ - 1 - window);
      // pass 1: the row's maximum over this tile; the whole row comes into registers at once (four
      // loads in flight, one wait) and is dropped again (only tiles on the diagonal or the window's
      // edge need the mask)
      float mx = -INFINITY;
      {
        constexpr int kChunks = BKV / 32;
        uint32_t sc[kChunks][32];
#pragma unroll
        for (int c = 0; c < kChunks; ++c) tmem_load32_async(my_s + c * 32, sc[c]);
        tmem_load_wait();
#pragma unroll
        for (int c = 0; c < kChunks; ++c) tmem_pin(sc[c]);
        if (edge) {
#pragma unroll
          for (int c = 0; c < kChunks; ++c)
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              const int key = key0 + c * 32 + e;
              if (key <= row && (window <= 0 || key > row - window)) mx = fmaxf(mx, __uint_as_float(sc[c][e]));
            }
        } else {
#pragma unroll
          for (int c = 0; c < kChunks; ++c)
#pragma unroll
            for (int e = 0; e < 32; ++e) mx = fmaxf(mx, __uint_as_float(sc[c][e]));
        }
      }
      m_run = fmaxf(m_run, mx * scale_log2);
      // bring O and the mass to the new maximum only when it has moved far (always for the first
      // tile, where O holds nothing yet and only the reference is set)
      const bool far = m_run > m_ref + kRescaleStep;
      if (j == 0) {
        m_ref = m_run;
      } else if (__any_sync(0xffffffffu, far)) {
        const float alpha = far ? fast_exp2(m_ref - m_run) : 1.0f;  // m_ref = -inf gives 0, and O is 0 then
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          tmem_load32(my_o + c * 32, r);
#pragma unroll
          for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * alpha);
          tmem_store32(my_o + c * 32, r);
        }
        tmem_store_wait();
        l *= alpha;
        if (far) m_ref = m_run;
      }
      const float m_use = m_ref == -INFINITY ? 0.f : m_ref;  // a row that has seen no key yet
      // pass 2: probabilities against m_ref, rounded to bfloat16, written over the scores they came
      // from: keys 32 c .. 32 c + 31 become columns 16 c .. 16 c + 15 (read by then). The next
      // chunk of scores is on its way while this one is worked on.
      float sum = 0.f;
      uint32_t sc[2][32];
      tmem_load32_async(my_s, sc[0]);
#pragma unroll
      for (int c = 0; c < BKV / 32; ++c) {
        tmem_load_wait();
        tmem_pin(sc[c & 1]);
        if (c + 1 < BKV / 32) tmem_load32_async(my_s + (c + 1) * 32, sc[(c + 1) & 1]);
        uint32_t packed[16];
        if (edge) {
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            const int key = key0 + c * 32 + e;
            const bool v0 = key <= row && (window <= 0 || key > row - window);
            const bool v1 = key + 1 <= row && (window <= 0 || key + 1 > row - window);
            const float p0 = v0 ? fast_exp2(fmaf(__uint_as_float(sc[c & 1][e]), scale_log2, -m_use)) : 0.f;
            const float p1 = v1 ? fast_exp2(fmaf(__uint_as_float(sc[c & 1][e + 1]), scale_log2, -m_use)) : 0.f;
            sum += p0 + p1;
            packed[e >> 1] = pack_bf16(p0, p1);
          }
        } else {
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            const float p0 = fast_exp2(fmaf(__uint_as_float(sc[c & 1][e]), scale_log2, -m_use));
            const float p1 = fast_exp2(fmaf(__uint_as_float(sc[c & 1][e + 1]), scale_log2, -m_use));
            sum += p0 + p1;
            packed[e >> 1] = pack_bf16(p0, p1);
          }
        }
        tmem_store16(my_s + c * 16, packed);
      }
      tmem_store_wait();
      l += sum;
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready + i);
    }
    if (ok && n_mine > 0) {
      if (!mbar_wait(o_done + i, 0, status, kStuckOutput)) {
        *bail = 1;
        ok = false;
      }
      tc_fence_after();
    }
    if (ok && n_mine > 0) {
      // the mass belongs to m_ref, and so does O: their quotient is the row's attention output
      const float inv = 1.0f / l;
      __nv_bfloat16* dst = out + (static_cast<size_t>(start + row) * q_heads + h) * D;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        tmem_load32(my_o + c * 32, r);
        if (row < len) {
#pragma unroll
          for (int e = 0; e < 32; e += 8)
            *reinterpret_cast<uint4*>(dst + c * 32 + e) = make_uint4(
                pack_bf16(__uint_as_float(r[e]) * inv, __uint_as_float(r[e + 1]) * inv),
                pack_bf16(__uint_as_float(r[e + 2]) * inv, __uint_as_float(r[e + 3]) * inv),
                pack_bf16(__uint_as_float(r[e + 4]) * inv, __uint_as_float(r[e + 5]) * inv),
                pack_bf16(__uint_as_float(r[e + 6]) * inv, __uint_as_float(r[e + 7]) * inv));
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kIssuerWarp) tmem_dealloc(tmem_base, kTmemColumns);
}

template <int D, int NQ, int BKV = 128>
int launch(const void* q, const void* k, const void* v, void* out, const int* cu_seqlens, int tokens,
           int seqs, int max_seq_len, int q_heads, int kv_heads, float scale, int window, int* status,
           cudaStream_t stream) {
  CUtensorMap map_q, map_k, map_v;
  if (!make_map_bf16(&map_q, q, tokens, static_cast<long long>(q_heads) * D, BQ) ||
      !make_map_bf16(&map_k, k, tokens, static_cast<long long>(kv_heads) * D, BKV) ||
      !make_map_bf16(&map_v, v, tokens, static_cast<long long>(kv_heads) * D, BKV))
    return LRM_UNSUPPORTED;
  constexpr int smem = NQ * BQ * D * 2 + 2 * Shape<D, BKV>::kStages * BKV * D * 2 + 256;
  auto kernel = attention_prefill_pingpong_kernel<D, NQ, BKV>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return static_cast<int>(e);
  const int pairs = (max_seq_len + NQ * BQ - 1) / (NQ * BQ);
  if (seqs > 65535 || pairs > 65535) return LRM_UNSUPPORTED;
  const dim3 grid(q_heads, seqs, pairs);
  LRM_LAUNCH(kernel, grid, dim3(threads_per_cta(NQ)), smem, stream, map_q, map_k, map_v,
             static_cast<__nv_bfloat16*>(out), cu_seqlens, q_heads, kv_heads, scale * 1.4426950408889634f, window,
             status);
  return 0;
}

}  // namespace

LRM_API int lrm_attention_prefill_pingpong_supports(int head_dim) {
  return (head_dim == 64 || head_dim == 128) && encode_tiled() != nullptr ? 1 : 0;
}

// q [tokens, q_heads, d], k, v [tokens, kv_heads, d] packed bfloat16, 16-byte aligned; `status`: one
// int in device memory, 0 before the launch; a kernel that gave up on a wait writes a code there.
LRM_API int lrm_attention_prefill_pingpong(const void* q, const void* k, const void* v, void* out,
                                           const int* cu_seqlens, int tokens, int seqs, int max_seq_len,
                                           int q_heads, int kv_heads, int d, float scale, int window,
                                           int* status, cudaStream_t stream) {
  if (seqs <= 0 || max_seq_len <= 0 || tokens <= 0) return 0;
  if (q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads != 0 || status == nullptr) return LRM_BAD_ARGUMENT;
  if (q_heads > 65535 || seqs > 65535) return LRM_UNSUPPORTED;
  if (reinterpret_cast<uintptr_t>(q) % 16 || reinterpret_cast<uintptr_t>(k) % 16 ||
      reinterpret_cast<uintptr_t>(v) % 16 || reinterpret_cast<uintptr_t>(out) % 16)
    return LRM_UNSUPPORTED;
  // Two query tiles per CTA where the head is wide (the tensor core then has work to hide a tile's
  // softmax under). With head size 64 one query tile per CTA, key tiles of 64 and four CTAs per SM:
  // the kernel is bound by the latency of its chain of dependent steps per key tile, and four
  // chains per SM hide more of it than two (measured against key tiles of 128 and two CTAs per SM:
  // 681 against 585 TFLOP/s at 32,768 tokens, 125 against 153 us at 4,096, four prompts of 512
  // tokens 20 against 29 us; two query tiles per CTA are slower at every length). Cutting a long
  // query tile's key tiles among several CTAs that meet through global memory (the last to arrive
  // adding the partials up) was measured as well: a single prompt of 2,048 tokens, whose longest
  // chain of 32 key tiles sets its time, took 67 us instead of 51 with chains of at most 17, and
  // more the shorter the chains.
  if (d == 64)
    return launch<64, 1, 64>(q, k, v, out, cu_seqlens, tokens, seqs, max_seq_len, q_heads, kv_heads, scale, window,
                         status, stream);
  // Head size 128: up to 2,304 tokens one query tile per CTA, key tiles of 64 and two CTAs per SM
  // (four prompts of 512 tokens 33 against 42 us, one of 2,048 tokens 61 against 63); beyond, two
  // query tiles per CTA taking turns (954 against 790 TFLOP/s at 32,768 tokens).
  if (d == 128 && max_seq_len <= 2304)
    return launch<128, 1, 64>(q, k, v, out, cu_seqlens, tokens, seqs, max_seq_len, q_heads, kv_heads, scale, window,
                              status, stream);
  if (d == 128)
    return launch<128, 2>(q, k, v, out, cu_seqlens, tokens, seqs, max_seq_len, q_heads, kv_heads, scale, window,
                          status, stream);
  return LRM_UNSUPPORTED;
}
