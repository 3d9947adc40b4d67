// bfloat16 matrix product on the 5th-generation tensor cores:
//   D[M,N] = X[M,K] . W[N,K]^T, float32 accumulation in tensor memory.
//
// A persistent kernel, one CTA per SM, each working through (128 MT) x BN tiles.
// Operand tiles (128 MT x 64 of X, BN x 64 of W, 128-byte swizzle) are brought
// into a ring of shared-memory stages by TMA (cp.async.bulk.tensor) issued by
// one thread; one other thread issues tcgen05.mma (M 128, N = BN, K 16) from
// shared-memory descriptors into TMEM accumulators of BN columns, MT of them per tile
// (one per 128 rows, sharing the W tile: a 256 x 256 tile needs a third less operand traffic
// from L2 per product than a 128 x 256 one, and that traffic is what bounds these products);
// with MT BN <= 256 two sets of accumulators alternate;
// tcgen05.commit signals both "stage free" to the loader and "accumulator
// ready" to the epilogue. Eight epilogue warps read their 32 TMEM lanes
// (tcgen05.ld, one row and half of its columns per thread) while the next tile's MMAs fill the
// other accumulator, and apply the epilogue:
//   0 store bfloat16, 1 store float32, 2 add into float32 in place (residual
//   stream), 3 SiLU gate over alternating blocks of 8 gate / 8 up columns,
//   4 store float32 partials per K slice.
// Rows and columns beyond M, N, K are zero-filled by TMA and skipped on store,
// so any M, N and any K that is a multiple of 8 is accepted.
// With `splits` > 1 (epilogue 4 only) an item covers a slice of K and stores its partial
// product in plane `slice` of an [splits, M, N] float32 tensor; whoever next reads the
// residual stream adds the planes in slice order (the norm kernel does it in its own pass).
// This is how a product with few rows and few columns (decode at batch 17-64: O and down
// projections) still fills the machine, with a result that does not depend on timing.
//
// Every wait on an mbarrier is bounded: after kSpinLimit polls the thread
// records where it gave up in `status` and the CTA winds down (waiting, again
// bounded, for its own copies in flight, then freeing its tensor memory).
// No cluster multicast is used anywhere.
// (Reference role: the tiled simdgroup GEMM,
// crates/metal-backend/src/shaders/matrix.metal:236-282.)
#include "gemm_epilogue.cuh"

namespace {

constexpr int BM = 128, BK = 64, UMMA_K = 16;

constexpr int kUmmaThreads = 320;  // loader warp, issuer warp, eight epilogue warps

// status codes (where a wait gave up)
enum : int { kStuckEmpty = 1, kStuckFull = 2, kStuckAccumulator = 3, kStuckDrain = 4, kStuckTmemFree = 5 };

// Persistent: CTA b works on items b, b + gridDim.x, ...; an item is (K slice, column tile, row
// tile) with the row tile fastest, so CTAs that run together share a tile of W in L2.
// Warp 0: TMA loader. Warp 1: MMA issuer (and owner of the tensor memory). Warps 2-9: epilogue.
// Where two sets of accumulators fit in the 512 columns of tensor memory they alternate, so the
// epilogue of one item runs under the MMAs of the next; a 256 x 256 tile fills it alone.
template <int BN, int STAGES, int MT>
__global__ __launch_bounds__(kUmmaThreads, 1) void gemm_bf16_umma_kernel(
    const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
    void* __restrict__ out, int M, int N, int K, int mode, int kb_per_split, int splits,
    int* __restrict__ status, const QkvArgs qkv) {
  constexpr uint32_t A_BYTES = MT * BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t SET = MT * BN;                      // columns of one set of accumulators
  constexpr uint32_t NBUF = 2 * SET <= 512 ? 2 : 1;      // sets that fit in tensor memory
  // tensor memory is handed out in powers of two of at least 32 columns (any other count is an
  // illegal instruction)
  constexpr uint32_t ALLOC = NBUF * SET <= 32 ? 32 : NBUF * SET <= 64 ? 64 : NBUF * SET <= 128 ? 128
                             : NBUF * SET <= 256 ? 256 : 512;
  static_assert(NBUF * SET <= 512, "accumulators do not fit in tensor memory");
  pdl_trigger();  // the next kernel may be scheduled as soon as an SM has room; it waits where it must
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // operand ring first (1024-byte aligned for the swizzle), then barriers
  unsigned char* tiles = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(tiles + STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;   // [2] accumulators written
  uint64_t* acc_free = acc_full + 2;     // [2] accumulators read back by all four epilogue warps
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_free + 2);
  volatile int* bail = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (M + MT * BM - 1) / (MT * BM), n_tiles = (N + BN - 1) / BN;
  const int items = m_tiles * n_tiles * splits;
  const int k_blocks = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(acc_full + a, 1);
      mbar_init(acc_free + a, 8);
    }
    *bail = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, ALLOC);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Barriers and tensor memory are set up while the kernel before this one may still run; what it
  // produced (X, and `out` where the epilogue adds) is touched only after the wait.
  pdl_wait();

  if (warp == 0) {
    if (lane == 0) {
      // ---- loader: one thread feeds the ring with TMA, straight through all items
      uint32_t it = 0;  // k blocks issued so far by this CTA
      for (int item = blockIdx.x; item < items && !*bail; item += gridDim.x) {
        const int m0 = (item % m_tiles) * MT * BM, n0 = ((item / m_tiles) % n_tiles) * BN;
        const int kb_begin = (item / (m_tiles * n_tiles)) * kb_per_split;
        const int num_kb = min(k_blocks - kb_begin, kb_per_split);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t round = it / STAGES;
          if (round > 0 && !mbar_wait(empty + s, (round - 1) & 1, status, kStuckEmpty)) {
            *bail = 1;
            break;
          }
          mbar_expect_tx(full + s, STAGE_BYTES);
#pragma unroll
          for (int i = 0; i < MT; ++i)  // 128 rows of X per accumulator (rows beyond M read as zero)
            tma_load_2d(tiles + s * STAGE_BYTES + i * BM * BK * 2, &map_x, full + s, (kb_begin + kb) * BK,
                        m0 + i * BM);
          tma_load_2d(tiles + s * STAGE_BYTES + A_BYTES, &map_w, full + s, (kb_begin + kb) * BK, n0);
        }
      }
      if (*bail) {
        // wait (bounded) for the copies already in flight before the CTA may exit
        const uint32_t first = it > STAGES ? it - STAGES : 0;
        for (uint32_t i = first; i < it; ++i)
          mbar_wait(full + i % STAGES, (i / STAGES) & 1, status, kStuckDrain);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- issuer: one thread drives the tensor core
      constexpr uint32_t idesc = umma_idesc(BM, BN);  // both operands K-major
      uint32_t it = 0, local = 0;
      for (int item = blockIdx.x; item < items && !*bail; item += gridDim.x, ++local) {
        const int kb_begin = (item / (m_tiles * n_tiles)) * kb_per_split;
        const int num_kb = min(k_blocks - kb_begin, kb_per_split);
        const uint32_t acc = local % NBUF, use = local / NBUF;
        // the epilogue must have emptied these accumulators (their previous use)
        if (use > 0 && !mbar_wait(acc_free + acc, (use - 1) & 1, status, kStuckTmemFree)) {
          *bail = 1;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * SET;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(full + s, (it / STAGES) & 1, status, kStuckFull)) {
            *bail = 1;
            break;
          }
          tc_fence_after();
          const uint32_t a = smem_u32(tiles + s * STAGE_BYTES), b = a + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
#pragma unroll
            for (int i = 0; i < MT; ++i)  // the 128-row blocks of X share the tile of W
              umma_bf16(tmem_d + i * BN, smem_desc(a + i * BM * BK * 2 + k * UMMA_K * 2),
                        smem_desc(b + k * UMMA_K * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(empty + s);  // arrives when these MMAs have finished reading the stage
        }
        umma_commit(acc_full + acc);  // arrives when every MMA issued so far has completed
      }
    }
  } else {
    // ---- epilogue: eight warps, one accumulator row per thread and half of its columns; a warp
    // may touch only the quarter of the tensor memory's lanes given by its index modulo 4
    const int quarter = warp & 3, side = (warp - 2) >> 2;
    uint32_t local = 0;
    for (int item = blockIdx.x; item < items; item += gridDim.x, ++local) {
      const int m0 = (item % m_tiles) * MT * BM, n0 = ((item / m_tiles) % n_tiles) * BN;
      const int kb_begin = (item / (m_tiles * n_tiles)) * kb_per_split;
      const int num_kb = min(k_blocks - kb_begin, kb_per_split);
      const uint32_t acc = local % NBUF, use = local / NBUF;
      if (*bail || !mbar_wait(acc_full + acc, use & 1, status, kStuckAccumulator)) {
        *bail = 1;
        break;
      }
      tc_fence_after();
      // epilogue 4: slice s owns plane s of `out` (the host never makes an empty slice)
      void* plane = mode == 4 ? static_cast<void*>(static_cast<float*>(out) +
                                                   static_cast<size_t>(item / (m_tiles * n_tiles)) * M * N)
                              : out;
      if (mode == 5) {  // whole heads of a q|k|v projection: rotate, store packed and into the cache
        // the first of the two warps of a row takes the first half of the tile's heads (rounded up)
        const int heads = BN / qkv.head_dim, cut = ((heads + 1) >> 1) * qkv.head_dim;
#pragma unroll 1
        for (int i = 0; i < MT; ++i)
          store_heads<BN>(tmem_base + acc * SET + i * BN + (static_cast<uint32_t>(quarter * 32) << 16),
                          m0 + i * BM + quarter * 32 + lane, n0, M, N, qkv, side == 0 ? 0 : cut, side == 0 ? cut : BN);
      } else if (num_kb > 0) {
        constexpr int kPieces = MT * BN / 32;
#pragma unroll 1
        for (int c = side * (kPieces / 2); c < (side + 1) * (kPieces / 2); ++c) {  // accumulator c / (BN / 32) holds rows 128 (c / (BN / 32)) ...
          const int m = m0 + (c / (BN / 32)) * BM + quarter * 32 + lane;
          uint32_t r[32];
          tmem_load32(tmem_base + acc * SET + (static_cast<uint32_t>(quarter * 32) << 16) + c * 32, r);
          store_piece(r, plane, m, n0 + (c % (BN / 32)) * 32, M, N, mode);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_free + acc);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, ALLOC);
}

// ------------------------------------------------------------------------- host side
template <int BN, int STAGES, int MT = 1>
int launch_umma(const void* X, const void* W, void* out, int M, int x_rows, int N, int K, int mode, int splits,
                int* status, cudaStream_t stream, const QkvArgs& qkv = QkvArgs{}) {
  CUtensorMap map_x, map_w;
  if (!make_map_bf16(&map_x, X, x_rows, K, BM) || !make_map_bf16(&map_w, W, N, K, BN)) return LRM_UNSUPPORTED;
  constexpr int smem = STAGES * (MT * BM * BK * 2 + BN * BK * 2) + 1024 + 256;
  auto kernel = gemm_bf16_umma_kernel<BN, STAGES, MT>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return static_cast<int>(e);
  const int k_blocks = (K + BK - 1) / BK;
  const int kb_per_split = (k_blocks + splits - 1) / splits;
  const int real_splits = (k_blocks + kb_per_split - 1) / kb_per_split;
  const long long items = static_cast<long long>((N + BN - 1) / BN) * ((M + MT * BM - 1) / (MT * BM)) * real_splits;
  static int sm_count = 0;
  if (sm_count == 0) {
    int device = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device);
    if (sm_count <= 0) sm_count = 148;
  }
  const int grid = static_cast<int>(items < sm_count ? items : sm_count);
  LRM_LAUNCH(kernel, dim3(grid), kUmmaThreads, smem, stream, map_x, map_w, out, M, N, K, mode, kb_per_split, real_splits,
             status, qkv);
  return 0;
}

}  // namespace

// Planes that epilogue 4 writes when K is cut into `splits` slices (no slice is ever empty).
LRM_API int lrm_gemm_bf16_umma_slices(int K, int splits) {
  if (K <= 0 || splits <= 1) return 1;
  const int k_blocks = (K + BK - 1) / BK;
  const int kb_per_split = (k_blocks + splits - 1) / splits;
  return (k_blocks + kb_per_split - 1) / kb_per_split;
}

// Shapes the tensor-core kernel takes: K a multiple of 8 (TMA needs 16-byte row pitches).
LRM_API int lrm_gemm_bf16_umma_supports(int M, int N, int K) {
  return M >= 1 && N >= 1 && K >= 8 && K % 8 == 0 && encode_tiled() != nullptr ? 1 : 0;
}

// `status`: one int in device memory, 0 before the launch; a kernel that gave up on a wait
// writes a nonzero code there (the result is then invalid and the caller must raise).
// `splits` > 1 cuts K into slices whose partial products go to the planes of an
// [lrm_gemm_bf16_umma_slices(K, splits), M, N] float32 tensor (epilogue 4 only).
// `tile`: 0 = 128 x 128, 1 = 128 x 256, 2 = 256 x 256, 3 = 128 x 192 (rows x columns of the output
// per item; the last one exists for products whose tiles would otherwise fill the SMs one and a
// bit times over).
// `x_rows` >= M: rows of X that may be read (the tensor map is built over them; rows from M on only
// feed accumulator rows that are never stored). TMA was measured slower on maps of fewer than 32
// rows, so a caller whose buffer holds 32 rows says so.
LRM_API int lrm_gemm_bf16_umma_rows(const void* X, const void* W, void* out, int M, int x_rows, int N, int K,
                                    int mode, int tile, int splits, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (!lrm_gemm_bf16_umma_supports(M, N, K)) return LRM_UNSUPPORTED;
  if (mode < 0 || mode > 4 || (mode == 3 && N % 16 != 0) || status == nullptr) return LRM_BAD_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(X) % 16 || reinterpret_cast<uintptr_t>(W) % 16) return LRM_UNSUPPORTED;
  if (splits < 1 || splits > 64 || (splits > 1 && mode != 4)) return LRM_BAD_ARGUMENT;
  if (tile < 0 || tile > 3) return LRM_BAD_ARGUMENT;
  if (x_rows < M) return LRM_BAD_ARGUMENT;
  if (tile == 3) return launch_umma<192, 5>(X, W, out, M, x_rows, N, K, mode, splits, status, stream);
  if (tile == 2) return launch_umma<256, 3, 2>(X, W, out, M, x_rows, N, K, mode, splits, status, stream);
  if (tile == 1) return launch_umma<256, 4>(X, W, out, M, x_rows, N, K, mode, splits, status, stream);
  return launch_umma<128, 6>(X, W, out, M, x_rows, N, K, mode, splits, status, stream);
}

// Epilogue 5: X . W^T is a prompt's fused q|k|v projection; it is rotated and stored as rope_store.cu
// would store it (see QkvArgs), without a launch of its own. The tile's width must be a whole
// number of heads; head sizes 64 and 128; rotation of the whole head or none.
LRM_API int lrm_gemm_bf16_umma_qkv(const void* X, const void* W, int M, int N, int K, int tile, void* q, void* k,
                                   void* v, void* k_pages, void* v_pages, const int* dest_rows,
                                   const float* table, int q_heads, int kv_heads, int head_dim, int page_size,
                                   int* status, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (!lrm_gemm_bf16_umma_supports(M, N, K)) return LRM_UNSUPPORTED;
  if (status == nullptr || q == nullptr || k == nullptr || v == nullptr || (k_pages != nullptr && dest_rows == nullptr))
    return LRM_BAD_ARGUMENT;
  if ((head_dim != 64 && head_dim != 128) || N != (q_heads + 2 * kv_heads) * head_dim) return LRM_UNSUPPORTED;
  if (reinterpret_cast<uintptr_t>(X) % 16 || reinterpret_cast<uintptr_t>(W) % 16 ||
      reinterpret_cast<uintptr_t>(table) % 16)
    return LRM_UNSUPPORTED;
  const int width = tile == 0 ? 128 : tile == 3 ? 192 : 256;
  if (tile < 0 || tile > 3 || width % head_dim != 0) return LRM_BAD_ARGUMENT;
  const QkvArgs args{static_cast<__nv_bfloat16*>(q), static_cast<__nv_bfloat16*>(k), static_cast<__nv_bfloat16*>(v),
                     static_cast<__nv_bfloat16*>(k_pages), static_cast<__nv_bfloat16*>(v_pages), dest_rows,
                     reinterpret_cast<const float2*>(table), q_heads, kv_heads, head_dim, page_size};
  if (tile == 3) return launch_umma<192, 5>(X, W, nullptr, M, M, N, K, 5, 1, status, stream, args);
  if (tile == 2) return launch_umma<256, 3, 2>(X, W, nullptr, M, M, N, K, 5, 1, status, stream, args);
  if (tile == 1) return launch_umma<256, 4>(X, W, nullptr, M, M, N, K, 5, 1, status, stream, args);
  return launch_umma<128, 6>(X, W, nullptr, M, M, N, K, 5, 1, status, stream, args);
}

LRM_API int lrm_gemm_bf16_umma(const void* X, const void* W, void* out, int M, int N, int K, int mode,
                               int tile, int splits, int* status, cudaStream_t stream) {
  return lrm_gemm_bf16_umma_rows(X, W, out, M, M, N, K, mode, tile, splits, status, stream);
}
