// Decode attention in one launch: position rotation of q and the new k, the write of the
// new k and v into the paged cache, attention over the cache split over its pages, and the
// merge of the splits.
//
// One thread-block cluster per (sequence, kv head, group of 16 query heads); the cluster's
// CTAs take the sequence's 64-key pages in turn (CTA r: pages r, r + S, ...), each through a
// three-stage cp.async ring, and reduce their partial results through distributed shared
// memory: every CTA sends (acc, max, mass) per query head to the CTA that finishes that part of
// the output, into a region of its shared memory kept for nothing else; the cluster
// synchronises once, and each finishing CTA reads only its own shared memory:
// out = sum acc_i 2^(m_i-M) / sum l_i 2^(m_i-M). Nobody reads a peer's memory, so nobody has to
// wait before it leaves. Nothing goes through global memory between the split and the merge,
// and no second kernel runs. A cluster of one CTA writes its output without any of this.
//
// The step's fused q|k|v projection is the input. The CTA that owns the sequence's last page
// rotates the new k row, writes it and the v row to the cache and places both in its shared
// tile, so the first cache pages are in flight while q and the new row are rotated.
//
// Rotation as in rope_store.cu (reference: crates/metal-backend/src/shaders/attention.metal
// :3-25, split-half; the context is split the same way at :61-121): angle = float(position)
// * inv_freq[i] in float32, the same operations in the same order, so q and k are bit-equal
// to what the separate kernel produces.
//
// Head sizes 32, 64, 128; rotary a multiple of 32; page size 64; no window (the caller uses
// the separate kernels otherwise).
#include <cooperative_groups.h>

#include "attention_mma.cuh"

namespace cg = cooperative_groups;

namespace {

// Pages of the cp.async ring per CTA.
template <int D> constexpr int stages_of() { return D == 128 ? 2 : 3; }

// The cluster's barrier in two halves: everybody arrives early and waits where it first needs the
// others (all threads of every CTA execute both).
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

// Rotate the query fragments in registers: columns c < SPAN * 16 pair with c + SPAN * 16, which
// the same thread holds in fragment ks + SPAN. Same operations as rope_store.cu.
template <int D, int SPAN>
__device__ __forceinline__ void rotate_q(uint32_t (&qa)[D / 16][4], const float* cs_tab, const float* sn_tab) {
  if constexpr (2 * SPAN <= D / 16) {
    const int t = threadIdx.x & 3;
#pragma unroll
    for (int ks = 0; ks < SPAN; ++ks) {
#pragma unroll
      for (int r = 0; r < 4; ++r) {  // register r: row g + 8 (r & 1), columns 16 ks + 8 (r >> 1) + 2t + {0, 1}
        const int c = 16 * ks + 8 * (r >> 1) + 2 * t;
        const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&qa[ks][r]);
        const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&qa[ks + SPAN][r]);
        const float xa0 = __bfloat162float(lo.x), xa1 = __bfloat162float(lo.y);
        const float xb0 = __bfloat162float(hi.x), xb1 = __bfloat162float(hi.y);
        const float c0 = cs_tab[c], s0 = sn_tab[c], c1 = cs_tab[c + 1], s1 = sn_tab[c + 1];
        qa[ks][r] = pack_bf16(fmaf(xa0, c0, -__fmul_rn(xb0, s0)), fmaf(xa1, c1, -__fmul_rn(xb1, s1)));
        qa[ks + SPAN][r] = pack_bf16(fmaf(xa0, s0, __fmul_rn(xb0, c0)), fmaf(xa1, s1, __fmul_rn(xb1, c1)));
      }
    }
  }
}

template <int D>
__global__ __launch_bounds__(kThreads) void attention_decode_cluster_kernel(
    const __nv_bfloat16* __restrict__ qkv, const int* __restrict__ positions,
    const float* __restrict__ inv_freq, int rotary, __nv_bfloat16* __restrict__ k_pages,
    __nv_bfloat16* __restrict__ v_pages, const int* __restrict__ dest_rows,
    __nv_bfloat16* __restrict__ out, const int* __restrict__ page_table, int table_stride,
    const int* __restrict__ slots, const int* __restrict__ kv_lens, int q_heads, int kv_heads,
    int row_groups, float scale_log2, const int* __restrict__ order) {
  constexpr int STRIDE = D + 8, TILE = kTile * STRIDE, PART = D + 2, kStages = stages_of<D>();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ float cs_tab[D / 2], sn_tab[D / 2];
  __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* Vs = Ks + kStages * TILE;
  cg::cluster_group cluster = cg::this_cluster();
  const int n_ranks = static_cast<int>(cluster.num_blocks());
  // This kernel never lets the next one be scheduled before its CTAs exit. With an early
  // griddepcontrol.launch_dependents (at the top, or after the last page) the output projection,
  // the norm and the gate/up product are scheduled one after the other while attention still runs
  // (each of them triggers at once): a 16-layer chain of whole layers at batch 8 then took 54 us
  // per layer instead of 37 with single-CTA clusters, and the whole decode step 0.97 ms instead of
  // 0.89 with clusters of 6.
  const int rank = static_cast<int>(cluster.block_rank());
  const int pair = blockIdx.x / n_ranks;
  const int rg = pair % row_groups;
  const int kh = (pair / row_groups) % kv_heads;
  const int b_slot = pair / (row_groups * kv_heads);
  const int b = order != nullptr ? order[b_slot] : b_slot;  // sequences in the order given (longest first)
  const int group = q_heads / kv_heads;
  const int head0 = kh * group + 16 * rg;          // first query head of this cluster
  const int rows = min(16, group - 16 * rg);       // query heads it owns
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;

  // Lengths, slots, destinations and the page table were set before the step.
  const int len = kv_lens[b];                      // keys including the new one
  const int n_pages = (len + kTile - 1) / kTile;
  const int n_mine = rank < n_pages ? (n_pages - rank + n_ranks - 1) / n_ranks : 0;
  const int* table = page_table + static_cast<size_t>(slots[b]) * table_stride;
  const bool owner = n_mine > 0 && rank + (n_mine - 1) * n_ranks == n_pages - 1;  // has the last page
  const int new_row = (len - 1) % kTile;

  const size_t qkv_row = static_cast<size_t>(q_heads + 2 * kv_heads) * D;
  const __nv_bfloat16* src = qkv + static_cast<size_t>(b) * qkv_row;
  uint32_t qa[D / 16][4];
  // A CTA's peers must have started before it writes into their shared memory: everybody arrives
  // here and waits just before the first such write, long after.
  if (n_ranks > 1) cluster_arrive();
  auto issue = [&](int i) {  // my i-th page into ring slot i % kStages (nothing if I have no such page)
    if (i < n_mine) {
      const int page_index = rank + i * n_ranks;
      const size_t page = static_cast<size_t>(table[page_index]);
      const size_t base = (page * kv_heads + kh) * kTile * D;
      const int stage = i % kStages;
      load_page<D>(Ks + stage * TILE, k_pages + base, len - page_index * kTile);
      load_page<D>(Vs + stage * TILE, v_pages + base, len - page_index * kTile);
    }
    cp_async_commit();
  };
  // The cache rows of earlier tokens do not depend on the kernel before this one (the wait
  // returns at once unless the launch was made a programmatic dependent).
#pragma unroll
  for (int i = 0; i < kStages - 1; ++i) issue(i);
  pdl_wait();

  // ---- rotation: table of cos/sin for this sequence's position, q fragments, the new k/v row
  const int half = rotary / 2;
  const bool rotate = inv_freq != nullptr && half > 0;
  if (rotate && threadIdx.x < half) {
    const float angle = __fmul_rn(static_cast<float>(positions[b]), inv_freq[threadIdx.x]);
    sincosf(angle, &sn_tab[threadIdx.x], &cs_tab[threadIdx.x]);
  }
  // the new key (a pair of elements per thread) and value (an element per thread), owner only
  float ka = 0.f, kb = 0.f;
  int ia = 0, ib = 0;
  __nv_bfloat16 v_new = __float2bfloat16_rn(0.f);
  if (owner) {
    const __nv_bfloat16* k_src = src + static_cast<size_t>(q_heads + kh) * D;
    if (threadIdx.x < D / 2) {
      const int i = threadIdx.x;
      if (rotate && i < half) {
        ia = i;
        ib = i + half;
      } else {
        ia = (rotate ? rotary : 0) + 2 * (i - (rotate ? half : 0));
        ib = ia + 1;
      }
      ka = __bfloat162float(k_src[ia]);
      kb = __bfloat162float(k_src[ib]);
    }
    if (threadIdx.x < D) v_new = src[static_cast<size_t>(q_heads + kv_heads + kh) * D + threadIdx.x];
  }
  load_q<D>(qa, src + static_cast<size_t>(head0) * D, D, rows);
  __syncthreads();  // the table is complete
  if (rotate) {
    // the partner of column c is column c + half: fragment ks + half / 16
    if (half == 16) rotate_q<D, 1>(qa, cs_tab, sn_tab);
    if (half == 32) rotate_q<D, 2>(qa, cs_tab, sn_tab);
    if (half == 48) rotate_q<D, 3>(qa, cs_tab, sn_tab);
    if (half == 64) rotate_q<D, 4>(qa, cs_tab, sn_tab);
    if (owner && threadIdx.x < half) {
      const float cs = cs_tab[threadIdx.x], sn = sn_tab[threadIdx.x];
      const float ya = fmaf(ka, cs, -__fmul_rn(kb, sn)), yb = fmaf(ka, sn, __fmul_rn(kb, cs));
      ka = ya;
      kb = yb;
    }
  }
  if (owner) {  // the new row goes to the cache for later steps (this step reads it from shared memory)
    const int dest = dest_rows[b];
    if (dest >= 0) {
      const size_t page = static_cast<size_t>(dest / kTile);
      const size_t at = ((page * kv_heads + kh) * kTile + dest % kTile) * D;
      if (threadIdx.x < D / 2) {
        k_pages[at + ia] = __float2bfloat16_rn(ka);
        k_pages[at + ib] = __float2bfloat16_rn(kb);
      }
      if (threadIdx.x < D) v_pages[at + threadIdx.x] = v_new;
    }
  }

  float o[D / 8][4];
#pragma unroll
  for (int dn = 0; dn < D / 8; ++dn)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[dn][e] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  for (int i = 0; i < n_mine; ++i) {
    const int stage = i % kStages;
    const int page_index = rank + i * n_ranks;
    cp_async_wait<kStages - 2>();     // all but the newest kStages - 2 groups: page i is here
    __syncthreads();                  // ... for every thread, and everyone is done with page i - 1
    issue(i + kStages - 1);           // into the slot page i - 1 was in
    if (page_index == n_pages - 1) {  // the owner's last page: put the new row where its tile expects it
      __nv_bfloat16* k_row = Ks + stage * TILE + new_row * STRIDE;
      __nv_bfloat16* v_row = Vs + stage * TILE + new_row * STRIDE;
      if (threadIdx.x < D / 2) {
        k_row[ia] = __float2bfloat16_rn(ka);
        k_row[ib] = __float2bfloat16_rn(kb);
      }
      if (threadIdx.x < D) v_row[threadIdx.x] = v_new;
      __syncthreads();
    }
    float s[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
    scores<D, 2>(s, qa, Ks + stage * TILE + 16 * warp * STRIDE);
    if ((page_index + 1) * kTile <= len) {  // a full page: every key counts
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[nt][e] *= scale_log2;
    } else {
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = page_index * kTile + 16 * warp + 8 * nt + 2 * t + (e & 1);
          s[nt][e] = key < len ? s[nt][e] * scale_log2 : -INFINITY;
        }
      }
    }
    if (rows > 8) softmax_update<D, 2, 2>(s, o, m, l);
    else softmax_update<D, 2, 1>(s, o, m, l);  // query heads 8..15 of the tile are padding
    weighted_values<D, 2>(o, s, Vs + stage * TILE + 16 * warp * STRIDE);
  }
  cp_async_wait<0>();  // only empty groups can be left

  // Combine the four warps (each saw 16 keys of every page) through shared memory, which the
  // K/V tiles no longer need: per warp [16 rows][D + 2] floats (acc, max, mass).
  __syncthreads();
  float* all = reinterpret_cast<float*>(smem_raw);
  {
    float* stage = all + warp * 16 * PART;
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      float total = l[hf];
      total += __shfl_xor_sync(0xffffffffu, total, 1);
      total += __shfl_xor_sync(0xffffffffu, total, 2);
      if (g + 8 * hf < rows) {
        float* dst = stage + (g + 8 * hf) * PART;
#pragma unroll
        for (int dn = 0; dn < D / 8; ++dn)
          *reinterpret_cast<float2*>(dst + 8 * dn + 2 * t) = make_float2(o[dn][2 * hf], o[dn][2 * hf + 1]);
        if (t == 0) {
          dst[D] = m[hf];
          dst[D + 1] = total;
        }
      }
    }
  }
  __syncthreads();
  if (n_ranks == 1) {  // nobody to meet: finish every output from the four warps' parts
    for (int item = threadIdx.x; item < rows * D; item += kThreads) {
      const int r = item / D, d = item % D;
      float mw[4], M = -INFINITY;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        mw[w] = all[(w * 16 + r) * PART + D];
        M = fmaxf(M, mw[w]);
      }
      float acc = 0.f, mass = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float weight = mw[w] == -INFINITY ? 0.f : exp2f(mw[w] - M);
        acc = fmaf(all[(w * 16 + r) * PART + d], weight, acc);
        mass = fmaf(all[(w * 16 + r) * PART + D + 1], weight, mass);
      }
      out[(static_cast<size_t>(b) * q_heads + head0 + r) * D + d] = __float2bfloat16_rn(acc / mass);
    }
    return;
  }

  // The outputs (row r, column d), numbered r * D + d, are finished in runs of 128: run j by CTA
  // j % n_ranks as its (j / n_ranks)-th. A row lies within one run (D divides 128), so its max and
  // mass go to one CTA. Every CTA sends each value of its partial to the CTA that finishes it:
  // received[sender][run][128] for the accumulators, then [sender][16 rows][max, mass].
  const int runs = (rows * D + 127) / 128;
  const int runs_each = (runs + n_ranks - 1) / n_ranks;
  float* received = reinterpret_cast<float*>(smem_raw + 2 * kStages * TILE * sizeof(__nv_bfloat16));
  const int ml_at = n_ranks * runs_each * 128;
  cluster_wait();  // every peer has started (all arrived at the top)
  for (int item = threadIdx.x; item < rows * PART; item += kThreads) {
    const int r = item / PART, c = item % PART;
    float mw[4], M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      mw[w] = all[(w * 16 + r) * PART + D];
      M = fmaxf(M, mw[w]);
    }
    float value;
    if (c == D) {
      value = M;
    } else {  // accumulator columns and the mass column scale alike
      value = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w)
        value += mw[w] == -INFINITY ? 0.f : all[(w * 16 + r) * PART + c] * exp2f(mw[w] - M);
    }
    const int number = r * D + (c < D ? c : 0);
    const int run = number >> 7;
    float* theirs = cluster.map_shared_rank(received, run % n_ranks);
    if (c < D) theirs[(rank * runs_each + run / n_ranks) * 128 + (number & 127)] = value;
    else theirs[ml_at + (rank * 16 + r) * 2 + (c - D)] = value;
  }
  cluster.sync();  // everything sent to me has arrived

  for (int mine = 0; mine < runs_each; ++mine) {
    const int number = ((mine * n_ranks + rank) << 7) + threadIdx.x;
    if (number >= rows * D) break;
    const int r = number / D;
    float M = -INFINITY;
    for (int u = 0; u < n_ranks; ++u) M = fmaxf(M, received[ml_at + (u * 16 + r) * 2]);
    float acc = 0.f, mass = 0.f;
    for (int u = 0; u < n_ranks; ++u) {  // a part that saw no key has max -inf and weight 0
      const float mu = received[ml_at + (u * 16 + r) * 2];
      const float weight = mu == -INFINITY ? 0.f : exp2f(mu - M);
      acc = fmaf(received[(u * runs_each + mine) * 128 + threadIdx.x], weight, acc);
      mass = fmaf(received[ml_at + (u * 16 + r) * 2 + 1], weight, mass);
    }
    out[(static_cast<size_t>(b) * q_heads + head0 + r) * D + (number % D)] = __float2bfloat16_rn(acc / mass);
  }
}

// Bytes of shared memory: the K/V ring, and for clusters the region that partials are sent into
// (n CTAs x (ceil(runs / n) x 128 accumulators + 16 rows x (max, mass))), for up to `rows` query
// heads per kv head in a CTA.
template <int D> int smem_bytes(int cluster, int rows) {
  const int ring = 2 * stages_of<D>() * kTile * (D + 8) * 2;
  if (cluster <= 1) return ring;
  const int runs = (rows * D + 127) / 128, runs_each = (runs + cluster - 1) / cluster;
  return ring + cluster * (runs_each * 128 + 32) * 4;
}


template <int D> int prepare(int cluster) {
  auto kernel = attention_decode_cluster_kernel<D>;
  int most = 0;  // over every cluster size and up to 16 query heads per kv head
  for (int c = 1; c <= 16; ++c) most = max(most, smem_bytes<D>(c, 16));
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (cluster > 8) {
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  return 0;
}

template <int D> void fill_config(cudaLaunchConfig_t& config, cudaLaunchAttribute* attributes, int pairs,
                                  int cluster, int rows, cudaStream_t stream) {
  config.gridDim = dim3(pairs * cluster);
  config.blockDim = dim3(kThreads);
  config.dynamicSmemBytes = smem_bytes<D>(cluster, rows);
  config.stream = stream;
  attributes[0].id = cudaLaunchAttributeClusterDimension;
  attributes[0].val.clusterDim.x = cluster;
  attributes[0].val.clusterDim.y = 1;
  attributes[0].val.clusterDim.z = 1;
  // Clusters of more than one CTA are launched without programmatic stream serialization:
  // started early as a dependent of the projection before it, the kernel made the whole decode
  // step 10-20 % slower (measured at batch 8, clusters of 6 and 8): its CTAs then start one by one
  // over 12 us, as that kernel's CTAs leave their SMs, and each still needs its own 12 us (three
  // dependent loads before the first page arrives, the pages, the meeting of the cluster), so the
  // last one ends later than if all had started together. Single-CTA clusters (large batches)
  // gain from the early start and keep it.
  attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attributes[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attributes;
  config.numAttrs = g_lrm_pdl && cluster == 1 ? 2 : 1;
}

// How many clusters of this size can be resident at once (0: this size cannot be launched).
template <int D> int resident_clusters(int cluster, int rows) {
  int code = prepare<D>(cluster);
  if (code != 0) return 0;
  cudaLaunchConfig_t config = {};
  cudaLaunchAttribute attributes[2];
  fill_config<D>(config, attributes, 1, cluster, rows, nullptr);
  config.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, attention_decode_cluster_kernel<D>, &config) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

template <int D> int launch(const void* qkv, const int* positions, const float* inv_freq, int rotary,
                            void* k_pages, void* v_pages, const int* dest_rows, void* out,
                            const int* page_table, int table_stride, const int* slots, const int* kv_lens,
                            int seqs, int q_heads, int kv_heads, float scale, int cluster,
                            cudaStream_t stream, const int* order = nullptr) {
  int code = prepare<D>(cluster);
  if (code != 0) return code;
  const int group = q_heads / kv_heads, row_groups = (group + 15) / 16;
  cudaLaunchConfig_t config = {};
  cudaLaunchAttribute attributes[2];
  fill_config<D>(config, attributes, seqs * kv_heads * row_groups, cluster, min(group, 16), stream);
  cudaError_t e = cudaLaunchKernelEx(
      &config, attention_decode_cluster_kernel<D>, static_cast<const __nv_bfloat16*>(qkv), positions,
      inv_freq, rotary, static_cast<__nv_bfloat16*>(k_pages), static_cast<__nv_bfloat16*>(v_pages),
      dest_rows, static_cast<__nv_bfloat16*>(out), page_table, table_stride, slots, kv_lens, q_heads,
      kv_heads, row_groups, scale * 1.4426950408889634f, order);
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

}  // namespace

// 1 when the fused decode kernel takes this geometry (bfloat16 only).
LRM_API int lrm_attention_decode_cluster_supports(int head_dim, int page_size, int rotary) {
  return (head_dim == 32 || head_dim == 64 || head_dim == 128) && page_size == kTile && rotary >= 0 &&
         rotary <= head_dim && rotary % 32 == 0;
}

// Clusters of `cluster` CTAs, each with `rows` (1-16) query heads per kv head, that fit on the device
// at once; 0 when that size cannot be launched.
LRM_API int lrm_attention_decode_cluster_resident(int head_dim, int cluster, int rows) {
  if (cluster < 1 || cluster > 16 || rows < 1 || rows > 16) return 0;
  if (head_dim == 32) return resident_clusters<32>(cluster, rows);
  if (head_dim == 64) return resident_clusters<64>(cluster, rows);
  if (head_dim == 128) return resident_clusters<128>(cluster, rows);
  return 0;
}

// qkv: [seqs, (q_heads + 2 kv_heads) * d] bfloat16, this step's fused projection, unrotated.
// positions, dest_rows, slots, kv_lens: int32 [seqs]; kv_lens counts the new token;
// dest_rows[b] = page * 64 + row where the new key/value row is stored. out: [seqs, q_heads, d].
// order: int32 [seqs] or nullptr: the sequences in the order their clusters are to start (the longest
// first: clusters beyond what the device holds at once then are those of the short sequences).
LRM_API int lrm_attention_decode_cluster(const void* qkv, const int* positions, const float* inv_freq,
                                         int rotary, void* k_pages, void* v_pages, const int* dest_rows,
                                         void* out, const int* page_table, int table_stride,
                                         const int* slots, const int* kv_lens, int seqs, int q_heads,
                                         int kv_heads, int head_dim, int page_size, float scale,
                                         int cluster, const int* order, cudaStream_t stream) {
  if (seqs <= 0) return 0;
  if (q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads != 0 || cluster < 1 || cluster > 16)
    return LRM_BAD_ARGUMENT;
  if (inv_freq == nullptr) rotary = 0;
  if (!lrm_attention_decode_cluster_supports(head_dim, page_size, rotary)) return LRM_UNSUPPORTED;
#define LRM_CASE(DIM)                                                                                  \
  if (head_dim == DIM)                                                                                 \
    return launch<DIM>(qkv, positions, inv_freq, rotary, k_pages, v_pages, dest_rows, out, page_table, \
                       table_stride, slots, kv_lens, seqs, q_heads, kv_heads, scale, cluster, stream, order);
  LRM_CASE(32)
  LRM_CASE(64)
  LRM_CASE(128)
#undef LRM_CASE
  return LRM_UNSUPPORTED;
}
