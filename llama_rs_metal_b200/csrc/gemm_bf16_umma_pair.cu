// bfloat16 matrix product on the 5th-generation tensor cores, two SMs per tile:
//   D[M,N] = X[M,K] . W[N,K]^T, float32 accumulation in tensor memory.
//
// What bounds the single-CTA kernel (gemm_bf16_umma.cu) on large products is operand traffic
// from L2 into an SM's shared memory: a 128 x 256 tile takes 48 KB per 64 of K. Here a cluster
// of two CTAs works on one 256 x 256 tile with tcgen05.mma.cta_group::2: CTA r of the pair loads
// rows [128 r, 128 r + 128) of the X tile and rows [128 r, 128 r + 128) of the W tile (32 KB per
// 64 of K and SM, a third less), the tensor cores of both SMs read both halves of W, and each
// CTA's tensor memory receives its 128 rows of the 256-column result. That leaves room for two
// sets of accumulators per CTA (2 x 256 columns), so a tile's epilogue runs under the next
// tile's MMAs, and for a ring of six stages.
//
// Who does what: in each CTA one thread issues the TMA loads of its halves; they complete on the
// leader's (CTA 0's) "full" barrier, which expects the bytes of both CTAs. One thread of the
// leader issues the MMAs for the pair and commits to the "stage free" and "accumulator ready"
// barriers of both CTAs (tcgen05.commit with a CTA mask). Eight epilogue warps per CTA read their
// CTA's accumulator rows and tell the leader's "accumulator free" barrier when done. Tensor
// memory is allocated and freed by one warp of each CTA together, as cta_group::2 requires.
// Epilogues as in the single-CTA kernel (0-3; K is never sliced here).
//
// Every wait on an mbarrier is bounded: after kSpinLimit polls the thread records where it gave
// up in `status` and its CTA winds down; both CTAs of a pair always meet at the cluster barrier
// at the end before the tensor memory is freed. The TMA loads carry no cluster multicast.
// (Reference role: the tiled simdgroup GEMM, crates/metal-backend/src/shaders/matrix.metal:236-282.)
#include "gemm_epilogue.cuh"

namespace {

constexpr int PM = 128, PK = 64, P_UMMA_K = 16;  // rows per CTA, K per stage, K per instruction
constexpr int kPairThreads = 320;                // loader warp, tensor-memory/issuer warp, eight epilogue warps

enum : int { kPairStuckEmpty = 31, kPairStuckFull = 32, kPairStuckAccumulator = 33, kPairStuckDrain = 34,
             kPairStuckTmemFree = 35 };

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// The address, in the cluster's shared window, of the same location in CTA `rank`.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
  return remote;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// A tile into this CTA's shared memory; the bytes are counted on the barrier at `bar_cluster`,
// which may belong to the other CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster, int x,
                                                 int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* dst, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst)),
               "r"(columns));
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::);
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t addr, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(columns));
}
// One arrival on the barrier at this offset in every CTA of `mask`, when all tcgen05 operations
// this thread issued so far are complete.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar, uint16_t mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)), "h"(mask)
      : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Pair p (CTAs 2p and 2p + 1) works on items p, p + pairs, ...; an item is a (column tile, row
// tile) of 256 rows x BN columns with the row tile fastest.
// Warp 0: TMA loader. Warp 1: tensor memory, and in the leader the MMA issuer. Warps 2-9: epilogue.
template <int BN, int STAGES>
__global__ __launch_bounds__(kPairThreads, 1) void gemm_bf16_umma_pair_kernel(
    const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
    void* __restrict__ out, int M, int N, int K, int mode, int* __restrict__ status, const QkvArgs qkv) {
  constexpr uint32_t A_BYTES = PM * PK * 2, B_BYTES = (BN / 2) * PK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t ALLOC = 512, SET = 256;  // two sets of accumulators, 256 columns apart
  static_assert(BN % 32 == 0 && BN >= 64 && BN <= 256, "BN / 2 rows of W per CTA, a multiple of 16");
  static_assert(B_BYTES % 1024 == 0, "stages must stay 1024-byte aligned for the swizzle");
  pdl_trigger();
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(tiles + STAGES * STAGE_BYTES);  // the leader's are used
  uint64_t* empty = full + STAGES;       // each CTA's own: the leader's MMAs have read the stage
  uint64_t* acc_full = empty + STAGES;   // [2] each CTA's own: accumulators written
  uint64_t* acc_free = acc_full + 2;     // [2] the leader's: read back by the epilogue warps of both CTAs
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_free + 2);
  volatile int* bail = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int m_tiles = (M + 2 * PM - 1) / (2 * PM), n_tiles = (N + BN - 1) / BN;
  const int items = m_tiles * n_tiles;
  const int k_blocks = (K + PK - 1) / PK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(acc_full + a, 1);
      mbar_init(acc_free + a, 16);  // eight epilogue warps in each of the two CTAs
    }
    *bail = 0;
    mbar_fence_init();
  }
  if (warp == 1) {  // the same warp of both CTAs, together
    tmem_alloc_pair(tmem_slot, ALLOC);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anything of mine reaches them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();

  if (warp == 0) {
    if (lane == 0) {
      // ---- loader: this CTA's half of the X rows and of the W rows of every stage
      uint32_t it = 0;
      for (int item = pair; item < items && !*bail; item += pairs) {
        const int m0 = (item % m_tiles) * 2 * PM + static_cast<int>(rank) * PM;
        const int n0 = (item / m_tiles) * BN + static_cast<int>(rank) * (BN / 2);
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t round = it / STAGES;
          if (round > 0 && !mbar_wait(empty + s, (round - 1) & 1, status, kPairStuckEmpty)) {
            *bail = 1;
            break;
          }
          if (leader) mbar_expect_tx(full + s, 2 * STAGE_BYTES);  // both CTAs' copies
          const uint32_t bar = map_to_rank(smem_u32(full + s), 0);
          tma_load_2d_pair(tiles + s * STAGE_BYTES, &map_x, bar, kb * PK, m0);
          tma_load_2d_pair(tiles + s * STAGE_BYTES + A_BYTES, &map_w, bar, kb * PK, n0);
        }
      }
      if (*bail && leader) {
        // wait (bounded) for the copies already in flight before the CTA may go on to exit
        const uint32_t first = it > STAGES ? it - STAGES : 0;
        for (uint32_t i = first; i < it; ++i)
          mbar_wait(full + i % STAGES, (i / STAGES) & 1, status, kPairStuckDrain);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      // ---- issuer: one thread of the leader drives the tensor cores of both SMs
      constexpr uint32_t idesc = umma_idesc(2 * PM, BN);
      uint32_t it = 0, local = 0;
      for (int item = pair; item < items && !*bail; item += pairs, ++local) {
        const uint32_t acc = local & 1, use = local >> 1;
        if (use > 0 && !mbar_wait(acc_free + acc, (use - 1) & 1, status, kPairStuckTmemFree)) {
          *bail = 1;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * SET;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(full + s, (it / STAGES) & 1, status, kPairStuckFull)) {
            *bail = 1;
            break;
          }
          tc_fence_after();
          const uint32_t a = smem_u32(tiles + s * STAGE_BYTES), b = a + A_BYTES;
#pragma unroll
          for (int k = 0; k < PK / P_UMMA_K; ++k)
            umma_bf16_pair(tmem_d, smem_desc(a + k * P_UMMA_K * 2), smem_desc(b + k * P_UMMA_K * 2), idesc,
                           (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit_pair(empty + s, 3);  // both CTAs' loaders may refill the stage
        }
        umma_commit_pair(acc_full + acc, 3);  // both CTAs' epilogues may read
      }
    }
  } else {
    // ---- epilogue: eight warps, one accumulator row and half of its columns per thread, this
    // CTA's 128 rows of the tile
    const int quarter = warp & 3, side = (warp - 2) >> 2;
    uint32_t local = 0;
    for (int item = pair; item < items; item += pairs, ++local) {
      const int m0 = (item % m_tiles) * 2 * PM + static_cast<int>(rank) * PM, n0 = (item / m_tiles) * BN;
      const uint32_t acc = local & 1, use = local >> 1;
      if (*bail || !mbar_wait(acc_full + acc, use & 1, status, kPairStuckAccumulator)) {
        *bail = 1;
        break;
      }
      tc_fence_after();
      if (mode == 5) {
        const int heads = BN / qkv.head_dim, cut = ((heads + 1) >> 1) * qkv.head_dim;
        store_heads<BN>(tmem_base + acc * SET + (static_cast<uint32_t>(quarter * 32) << 16),
                        m0 + quarter * 32 + lane, n0, M, N, qkv, side == 0 ? 0 : cut, side == 0 ? cut : BN);
      } else {
#pragma unroll 1
        for (int c = side * (BN / 64); c < (side + 1) * (BN / 64); ++c) {
          uint32_t r[32];
          tmem_load32(tmem_base + acc * SET + (static_cast<uint32_t>(quarter * 32) << 16) + c * 32, r);
          store_piece(r, out, m0 + quarter * 32 + lane, n0 + c * 32, M, N, mode);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_rank(smem_u32(acc_free + acc), 0));
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // nobody frees tensor memory or leaves while the other may still signal it
  if (warp == 1) tmem_dealloc_pair(tmem_base, ALLOC);
}

template <int BN, int STAGES> constexpr int pair_smem() {
  return STAGES * (PM * PK * 2 + (BN / 2) * PK * 2) + 1024 + 256;
}

template <int BN, int STAGES>
int pair_config(cudaLaunchConfig_t& config, cudaLaunchAttribute* attributes, int grid, cudaStream_t stream) {
  auto kernel = gemm_bf16_umma_pair_kernel<BN, STAGES>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, pair_smem<BN, STAGES>());
  if (e != cudaSuccess) return static_cast<int>(e);
  config.gridDim = dim3(grid);
  config.blockDim = dim3(kPairThreads);
  config.dynamicSmemBytes = pair_smem<BN, STAGES>();
  config.stream = stream;
  attributes[0].id = cudaLaunchAttributeClusterDimension;
  attributes[0].val.clusterDim.x = 2;
  attributes[0].val.clusterDim.y = 1;
  attributes[0].val.clusterDim.z = 1;
  attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attributes[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attributes;
  config.numAttrs = g_lrm_pdl ? 2 : 1;
  return 0;
}

// Pairs of CTAs the device runs at once (0: clusters of two cannot be launched).
template <int BN, int STAGES> int resident_pairs() {
  static int pairs = -1;
  if (pairs < 0) {
    cudaLaunchConfig_t config = {};
    cudaLaunchAttribute attributes[2];
    pairs = 0;
    if (pair_config<BN, STAGES>(config, attributes, 2, nullptr) == 0) {
      config.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, gemm_bf16_umma_pair_kernel<BN, STAGES>, &config) == cudaSuccess)
        pairs = n;
      else
        cudaGetLastError();
    }
  }
  return pairs;
}

template <int BN, int STAGES>
int launch_pair(const void* X, const void* W, void* out, int M, int N, int K, int mode, int* status,
                cudaStream_t stream, const QkvArgs& qkv = QkvArgs{}) {
  const int room = resident_pairs<BN, STAGES>();
  if (room <= 0) return LRM_UNSUPPORTED;
  CUtensorMap map_x, map_w;
  if (!make_map_bf16(&map_x, X, M, K, PM) || !make_map_bf16(&map_w, W, N, K, BN / 2)) return LRM_UNSUPPORTED;
  const long long items = static_cast<long long>((N + BN - 1) / BN) * ((M + 2 * PM - 1) / (2 * PM));
  const int pairs = static_cast<int>(items < room ? items : room);
  cudaLaunchConfig_t config = {};
  cudaLaunchAttribute attributes[2];
  int code = pair_config<BN, STAGES>(config, attributes, 2 * pairs, stream);
  if (code != 0) return code;
  cudaError_t e = cudaLaunchKernelEx(&config, gemm_bf16_umma_pair_kernel<BN, STAGES>, map_x, map_w, out, M, N, K,
                                     mode, status, qkv);
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

}  // namespace

// Pairs of SMs the two-CTA kernel can use at once; 0 when it cannot run on this device.
LRM_API int lrm_gemm_bf16_umma_pair_room() {
  if (encode_tiled() == nullptr) return 0;
  return resident_pairs<256, 6>();
}

// D = X . W^T with epilogue `mode` (0-3) in tiles of 256 x 256 over pairs of SMs. K a multiple of 8.
// (Tiles of 256 x 192 and 256 x 128 were measured too: a pair then needs as much operand traffic per
// product as a single CTA with a 128 x 256 tile, and only the QKV product of a 2,048-token prompt
// gained, 7 %.)
// `status` as for lrm_gemm_bf16_umma (codes 31-35 are this kernel's).
LRM_API int lrm_gemm_bf16_umma_pair(const void* X, const void* W, void* out, int M, int N, int K, int mode,
                                    int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K < 8 || K % 8 != 0 || encode_tiled() == nullptr) return LRM_UNSUPPORTED;
  if (mode < 0 || mode > 3 || (mode == 3 && N % 16 != 0) || status == nullptr) return LRM_BAD_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(X) % 16 || reinterpret_cast<uintptr_t>(W) % 16) return LRM_UNSUPPORTED;
  return launch_pair<256, 6>(X, W, out, M, N, K, mode, status, stream);
}

// Epilogue 5 on pairs of SMs (see lrm_gemm_bf16_umma_qkv): head sizes 64 and 128.
LRM_API int lrm_gemm_bf16_umma_pair_qkv(const void* X, const void* W, int M, int N, int K, void* q, void* k, void* v,
                                        void* k_pages, void* v_pages, const int* dest_rows, const float* table,
                                        int q_heads, int kv_heads, int head_dim, int page_size, int* status,
                                        cudaStream_t stream) {
  if (M <= 0) return 0;
  if (K < 8 || K % 8 != 0 || encode_tiled() == nullptr) return LRM_UNSUPPORTED;
  if (status == nullptr || q == nullptr || k == nullptr || v == nullptr || (k_pages != nullptr && dest_rows == nullptr))
    return LRM_BAD_ARGUMENT;
  if ((head_dim != 64 && head_dim != 128) || N != (q_heads + 2 * kv_heads) * head_dim) return LRM_UNSUPPORTED;
  if (reinterpret_cast<uintptr_t>(X) % 16 || reinterpret_cast<uintptr_t>(W) % 16 ||
      reinterpret_cast<uintptr_t>(table) % 16)
    return LRM_UNSUPPORTED;
  const QkvArgs args{static_cast<__nv_bfloat16*>(q), static_cast<__nv_bfloat16*>(k), static_cast<__nv_bfloat16*>(v),
                     static_cast<__nv_bfloat16*>(k_pages), static_cast<__nv_bfloat16*>(v_pages), dest_rows,
                     reinterpret_cast<const float2*>(table), q_heads, kv_heads, head_dim, page_size};
  return launch_pair<256, 6>(X, W, nullptr, M, N, K, 5, status, stream, args);
}
