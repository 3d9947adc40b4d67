// Causal grouped-query attention, one warp per (query, head), keys visited one
// at a time with a streaming softmax in float32:
//   s = (q.k) * scale;  m' = max(m, s);  l = l e^(m-m') + e^(s-m');
//   acc = acc e^(m-m') + e^(s-m') v;  out = acc / l
// (reference: crates/metal-backend/src/shaders/attention.metal:28-57).
// It is the attention of the float32 path for prompts and for decoding, and
// the bfloat16 path's fallback for sizes its tiled kernels refuse. The two
// entry points differ only in where keys come from (the step's packed k/v, or
// the paged cache), so a prompt, its token-by-token replay and its replay in
// chunks of any size do the same arithmetic in the same order. The paged entry
// takes any number of queries per sequence (a decoded token, or a portion of
// several tokens appended to a started sequence, whose own keys are already in
// the cache). A window w lets a query at position p see keys p-w+1 .. p.
#include "common.cuh"

constexpr int kMaxPerLane = 16;  // head_dim <= 512

struct PackedKeys {
  const void* k;
  const void* v;
  size_t base;  // index of the sequence's first packed token
  int kv_heads, d;
  template <typename A> __device__ const A* key(int p, int kh) const {
    return static_cast<const A*>(k) + ((base + p) * kv_heads + kh) * d;
  }
  template <typename A> __device__ const A* value(int p, int kh) const {
    return static_cast<const A*>(v) + ((base + p) * kv_heads + kh) * d;
  }
};

struct PagedKeys {
  const void* k;
  const void* v;
  const int* table;  // this slot's row of the page table
  int kv_heads, d, page_size;
  template <typename A> __device__ const A* key(int p, int kh) const {
    const size_t page = table[p / page_size];
    return static_cast<const A*>(k) + ((page * kv_heads + kh) * page_size + p % page_size) * d;
  }
  template <typename A> __device__ const A* value(int p, int kh) const {
    const size_t page = table[p / page_size];
    return static_cast<const A*>(v) + ((page * kv_heads + kh) * page_size + p % page_size) * d;
  }
};

template <typename A, typename Keys>
__device__ void attend_row(const A* __restrict__ q, A* __restrict__ out, const Keys& keys, int kh,
                           int first, int last, int d, float scale) {
  const int lane = threadIdx.x & 31;
  float qv[kMaxPerLane], acc[kMaxPerLane];
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    const int j = lane + 32 * i;
    qv[i] = j < d ? to_f32(q[j]) : 0.f;
    acc[i] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  for (int p = first; p <= last; ++p) {
    const A* kr = keys.template key<A>(p, kh);
    const A* vr = keys.template value<A>(p, kh);
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
      const int j = lane + 32 * i;
      if (j < d) dot = fmaf(qv[i], to_f32(kr[j]), dot);
    }
    const float s = warp_sum(dot) * scale;
    const float nm = fmaxf(m, s);
    const float old = expf(m - nm), prob = expf(s - nm);
    l = fmaf(l, old, prob);
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
      const int j = lane + 32 * i;
      if (j < d) acc[i] = fmaf(prob, to_f32(vr[j]), __fmul_rn(acc[i], old));
    }
    m = nm;
  }
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    const int j = lane + 32 * i;
    if (j < d) out[j] = from_f32<A>(acc[i] / l);
  }
}

template <typename A>
__global__ void attention_packed_kernel(const A* __restrict__ q, const A* __restrict__ k,
                                        const A* __restrict__ v, A* __restrict__ out,
                                        const int* __restrict__ cu_seqlens,
                                        const int* __restrict__ seq_of_token, int q_heads,
                                        int kv_heads, int d, float scale, int window) {
  const int t = blockIdx.x, h = blockIdx.y;
  const int start = cu_seqlens[seq_of_token[t]];
  const int pos = t - start;
  const int first = window > 0 ? max(0, pos - window + 1) : 0;
  PackedKeys keys{k, v, static_cast<size_t>(start), kv_heads, d};
  const size_t qo = (static_cast<size_t>(t) * q_heads + h) * d;
  attend_row<A>(q + qo, out + qo, keys, h / (q_heads / kv_heads), first, pos, d, scale);
}

template <typename A>
__global__ void attention_paged_kernel(const A* __restrict__ q, const A* __restrict__ k_pages,
                                       const A* __restrict__ v_pages, A* __restrict__ out,
                                       const int* __restrict__ page_table, int table_stride,
                                       const int* __restrict__ slots,
                                       const int* __restrict__ kv_lens,
                                       const int* __restrict__ seq_of_token,
                                       const int* __restrict__ positions, int q_heads, int kv_heads,
                                       int d, int page_size, float scale, int window) {
  // query t of the step belongs to sequence b and stands at position pos; without the two
  // arrays there is one query per sequence, its newest token
  const int t = blockIdx.x, h = blockIdx.y;
  const int b = seq_of_token != nullptr ? seq_of_token[t] : t;
  const int pos = positions != nullptr ? positions[t] : kv_lens[b] - 1;
  const int first = window > 0 ? max(0, pos - window + 1) : 0;
  PagedKeys keys{k_pages, v_pages, page_table + static_cast<size_t>(slots[b]) * table_stride,
                 kv_heads, d, page_size};
  const size_t qo = (static_cast<size_t>(t) * q_heads + h) * d;
  attend_row<A>(q + qo, out + qo, keys, h / (q_heads / kv_heads), first, pos, d, scale);
}

static bool bad_geometry(int q_heads, int kv_heads, int d) {
  return q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads != 0 || d <= 0 ||
         d > 32 * kMaxPerLane;
}

LRM_API int lrm_attention_packed_rowwise(const void* q, const void* k, const void* v, void* out,
                                         int dtype, const int* cu_seqlens, const int* seq_of_token,
                                         int tokens, int q_heads, int kv_heads, int d, float scale,
                                         int window, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (bad_geometry(q_heads, kv_heads, d)) return LRM_BAD_ARGUMENT;
  if (q_heads > 65535) return LRM_UNSUPPORTED;
  const dim3 grid(tokens, q_heads);
  if (dtype == LRM_F32)
    attention_packed_kernel<float><<<grid, 32, 0, stream>>>(
        static_cast<const float*>(q), static_cast<const float*>(k), static_cast<const float*>(v),
        static_cast<float*>(out), cu_seqlens, seq_of_token, q_heads, kv_heads, d, scale, window);
  else if (dtype == LRM_BF16)
    attention_packed_kernel<__nv_bfloat16><<<grid, 32, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k),
        static_cast<const __nv_bfloat16*>(v), static_cast<__nv_bfloat16*>(out), cu_seqlens,
        seq_of_token, q_heads, kv_heads, d, scale, window);
  else
    return LRM_BAD_ARGUMENT;
  LRM_LAUNCH_CHECK();
  return 0;
}

// `queries` rows of q. With seq_of_token and positions (int32 [queries]) query t belongs to
// sequence seq_of_token[t] and sees keys up to positions[t]; with both null there is one query
// per sequence, at position kv_lens[b] - 1.
LRM_API int lrm_attention_paged_rowwise(const void* q, const void* k_pages, const void* v_pages,
                                        void* out, int dtype, const int* page_table,
                                        int table_stride, const int* slots, const int* kv_lens,
                                        const int* seq_of_token, const int* positions,
                                        int queries, int q_heads, int kv_heads, int d, int page_size,
                                        float scale, int window, cudaStream_t stream) {
  if (queries <= 0) return 0;
  if (bad_geometry(q_heads, kv_heads, d) || page_size <= 0) return LRM_BAD_ARGUMENT;
  if ((seq_of_token == nullptr) != (positions == nullptr)) return LRM_BAD_ARGUMENT;
  if (positions == nullptr && kv_lens == nullptr) return LRM_BAD_ARGUMENT;
  if (q_heads > 65535) return LRM_UNSUPPORTED;
  const dim3 grid(queries, q_heads);
  if (dtype == LRM_F32)
    attention_paged_kernel<float><<<grid, 32, 0, stream>>>(
        static_cast<const float*>(q), static_cast<const float*>(k_pages),
        static_cast<const float*>(v_pages), static_cast<float*>(out), page_table, table_stride,
        slots, kv_lens, seq_of_token, positions, q_heads, kv_heads, d, page_size, scale, window);
  else if (dtype == LRM_BF16)
    attention_paged_kernel<__nv_bfloat16><<<grid, 32, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k_pages),
        static_cast<const __nv_bfloat16*>(v_pages), static_cast<__nv_bfloat16*>(out), page_table,
        table_stride, slots, kv_lens, seq_of_token, positions, q_heads, kv_heads, d, page_size, scale,
        window);
  else
    return LRM_BAD_ARGUMENT;
  LRM_LAUNCH_CHECK();
  return 0;
}
