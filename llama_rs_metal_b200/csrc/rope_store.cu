// Position rotation of q and k, and the write of k and v into the paged cache,
// in one pass over a step's fused q|k|v projection.
//
// Rotation (reference: crates/metal-backend/src/shaders/attention.metal:3-25,
// split-half branch): for pair i < R/2 of a head,
//   angle = float(position) * inv_freq[i]          (one float32 product)
//   y[i]       = x[i] cos - x[i + R/2] sin
//   y[i + R/2] = x[i] sin + x[i + R/2] cos
// dims >= R pass through; v is never rotated. inv_freq already holds the
// scaling (theta^(-2i/R) * scale / llama3 factor) and is built on the host.
// With inv_freq == nullptr nothing is rotated (another position scheme ran
// before, or none is used).
//
// Cache layout: pages [page][kv_head][page_size][d]. Where a token's key and
// value go is resolved on the host from the page table: dest_rows[t] =
// page * page_size + row in page, or < 0 when that position is not kept
// (outside a windowed group's window), which skips the store.
#include "common.cuh"

template <typename A>
__global__ void rope_store_kernel(const A* __restrict__ qkv, A* __restrict__ q_out,
                                  A* __restrict__ k_out, A* __restrict__ v_out,
                                  A* __restrict__ k_pages, A* __restrict__ v_pages,
                                  const int* __restrict__ dest_rows,
                                  const int* __restrict__ positions,
                                  const float* __restrict__ inv_freq, int rotary, int q_heads,
                                  int kv_heads, int d, int page_size) {
  pdl_trigger();  // a small kernel: let the next one start right away
  pdl_wait();
  const int t = blockIdx.x;
  const int first_item = blockIdx.y * blockDim.x, item_stride = gridDim.y * blockDim.x;
  const int pos = positions[t];
  const int half = rotary / 2, dh = d / 2;
  const size_t row = static_cast<size_t>(q_heads + 2 * kv_heads) * d;
  const A* src = qkv + static_cast<size_t>(t) * row;
  const int dest = k_pages != nullptr ? dest_rows[t] : -1;
  const long long page = dest >= 0 ? dest / page_size : -1;
  const int in_page = dest >= 0 ? dest % page_size : 0;
  const float fpos = static_cast<float>(pos);
  // rotated heads: q heads then k heads; one work item = one (head, i < d/2)
  const int rot_items = (q_heads + kv_heads) * dh;
  for (int item = first_item + threadIdx.x; item < rot_items; item += item_stride) {
    const int head = item / dh, i = item % dh;
    int a, b;  // the two elements this item produces
    float ya, yb;
    const A* x = src + static_cast<size_t>(head) * d;
    if (i < half) {
      a = i;
      b = i + half;
      const float xa = to_f32(x[a]), xb = to_f32(x[b]);
      if (inv_freq != nullptr) {
        const float angle = __fmul_rn(fpos, inv_freq[i]);
        float sn, cs;
        sincosf(angle, &sn, &cs);
        ya = fmaf(xa, cs, -__fmul_rn(xb, sn));
        yb = fmaf(xa, sn, __fmul_rn(xb, cs));
      } else {
        ya = xa;
        yb = xb;
      }
    } else {
      a = rotary + 2 * (i - half);
      b = a + 1;
      ya = to_f32(x[a]);
      yb = to_f32(x[b]);
    }
    const A oa = from_f32<A>(ya), ob = from_f32<A>(yb);
    if (head < q_heads) {
      A* dst = q_out + (static_cast<size_t>(t) * q_heads + head) * d;
      dst[a] = oa;
      dst[b] = ob;
    } else {
      const int kh = head - q_heads;
      if (k_out != nullptr) {
        A* dst = k_out + (static_cast<size_t>(t) * kv_heads + kh) * d;
        dst[a] = oa;
        dst[b] = ob;
      }
      if (page >= 0) {
        A* dst = k_pages + ((static_cast<size_t>(page) * kv_heads + kh) * page_size + in_page) * d;
        dst[a] = oa;
        dst[b] = ob;
      }
    }
  }
  // v heads: copy
  const A* vsrc = src + static_cast<size_t>(q_heads + kv_heads) * d;
  for (int item = first_item + threadIdx.x; item < kv_heads * d; item += item_stride) {
    const int kh = item / d, j = item % d;
    const A val = vsrc[item];
    if (v_out != nullptr) v_out[(static_cast<size_t>(t) * kv_heads + kh) * d + j] = val;
    if (page >= 0)
      v_pages[((static_cast<size_t>(page) * kv_heads + kh) * page_size + in_page) * d + j] = val;
  }
}

// The same work with 16-byte accesses: a thread takes VEC = 16 / sizeof(A) consecutive pairs
// (VEC elements of the first half and the VEC partners of the second half), a pass-through
// chunk, or a chunk of v. Needs R/2 and d to be multiples of VEC.
template <typename A> struct alignas(16) Vec16 { A v[16 / sizeof(A)]; };

template <typename A>
__global__ void rope_store_vec_kernel(const A* __restrict__ qkv, A* __restrict__ q_out,
                                      A* __restrict__ k_out, A* __restrict__ v_out,
                                      A* __restrict__ k_pages, A* __restrict__ v_pages,
                                      const int* __restrict__ dest_rows,
                                      const int* __restrict__ positions,
                                      const float* __restrict__ inv_freq, int rotary, int q_heads,
                                      int kv_heads, int d, int page_size) {
  constexpr int VEC = 16 / sizeof(A);
  using V = Vec16<A>;
  pdl_trigger();  // a small kernel: let the next one start right away
  pdl_wait();
  const int t = blockIdx.x;
  const int half = rotary / 2;
  const int rot_chunks = half / VEC, pass_chunks = (d - rotary) / VEC, v_chunks = d / VEC;
  const int heads = q_heads + kv_heads;
  const int n_rot = heads * rot_chunks, n_pass = heads * pass_chunks, n_v = kv_heads * v_chunks;
  const size_t row = static_cast<size_t>(q_heads + 2 * kv_heads) * d;
  const A* src = qkv + static_cast<size_t>(t) * row;
  const int pos = positions[t];
  const int dest = k_pages != nullptr ? dest_rows[t] : -1;
  const long long page = dest >= 0 ? dest / page_size : -1;
  const int in_page = dest >= 0 ? dest % page_size : 0;
  const float fpos = static_cast<float>(pos);

  // where element `e` of head `head` (q heads first, then k heads) goes
  auto store_qk = [&](int head, int e, const V& val) {
    if (head < q_heads) {
      *reinterpret_cast<V*>(q_out + (static_cast<size_t>(t) * q_heads + head) * d + e) = val;
    } else {
      const int kh = head - q_heads;
      if (k_out != nullptr)
        *reinterpret_cast<V*>(k_out + (static_cast<size_t>(t) * kv_heads + kh) * d + e) = val;
      if (page >= 0)
        *reinterpret_cast<V*>(k_pages + ((static_cast<size_t>(page) * kv_heads + kh) * page_size + in_page) * d + e) = val;
    }
  };

  for (int item = blockIdx.y * blockDim.x + threadIdx.x; item < n_rot + n_pass + n_v;
       item += gridDim.y * blockDim.x) {
    if (item < n_rot) {
      const int head = item / rot_chunks, c = item % rot_chunks;
      const A* x = src + static_cast<size_t>(head) * d;
      const V lo = *reinterpret_cast<const V*>(x + c * VEC);
      const V hi = *reinterpret_cast<const V*>(x + half + c * VEC);
      V out_lo, out_hi;
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        const float xa = to_f32(lo.v[e]), xb = to_f32(hi.v[e]);
        float ya = xa, yb = xb;
        if (inv_freq != nullptr) {
          const float angle = __fmul_rn(fpos, inv_freq[c * VEC + e]);
          float sn, cs;
          sincosf(angle, &sn, &cs);
          ya = fmaf(xa, cs, -__fmul_rn(xb, sn));
          yb = fmaf(xa, sn, __fmul_rn(xb, cs));
        }
        out_lo.v[e] = from_f32<A>(ya);
        out_hi.v[e] = from_f32<A>(yb);
      }
      store_qk(head, c * VEC, out_lo);
      store_qk(head, half + c * VEC, out_hi);
    } else if (item < n_rot + n_pass) {
      const int head = (item - n_rot) / pass_chunks, c = (item - n_rot) % pass_chunks;
      const int e = rotary + c * VEC;
      store_qk(head, e, *reinterpret_cast<const V*>(src + static_cast<size_t>(head) * d + e));
    } else {
      const int kh = (item - n_rot - n_pass) / v_chunks, c = (item - n_rot - n_pass) % v_chunks;
      const V val = *reinterpret_cast<const V*>(src + static_cast<size_t>(q_heads + kv_heads + kh) * d + c * VEC);
      if (v_out != nullptr)
        *reinterpret_cast<V*>(v_out + (static_cast<size_t>(t) * kv_heads + kh) * d + c * VEC) = val;
      if (page >= 0)
        *reinterpret_cast<V*>(v_pages + ((static_cast<size_t>(page) * kv_heads + kh) * page_size + in_page) * d + c * VEC) = val;
    }
  }
}

template <typename A>
static int launch_rope(const void* qkv, void* q_out, void* k_out, void* v_out, void* k_pages,
                       void* v_pages, const int* dest_rows, const int* positions,
                       const float* inv_freq, int rotary, int tokens, int q_heads, int kv_heads, int d,
                       int page_size, cudaStream_t stream) {
  constexpr int VEC = 16 / sizeof(A);
  auto aligned = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  const bool vec = d % VEC == 0 && (rotary / 2) % VEC == 0 && aligned(qkv) && aligned(q_out) &&
                   aligned(k_out) && aligned(v_out) && aligned(k_pages) && aligned(v_pages);
  if (vec) {
    const int work = (q_heads + kv_heads) * (d - rotary / 2) / VEC + kv_heads * d / VEC;
    const int threads = work >= 256 ? 256 : (work >= 128 ? 128 : 64);
    const dim3 grid(tokens, min(64, (work + threads - 1) / threads));
    LRM_LAUNCH(rope_store_vec_kernel<A>, grid, threads, 0, stream, static_cast<const A*>(qkv),
               static_cast<A*>(q_out), static_cast<A*>(k_out), static_cast<A*>(v_out),
               static_cast<A*>(k_pages), static_cast<A*>(v_pages), dest_rows, positions, inv_freq,
               rotary, q_heads, kv_heads, d, page_size);
    return 0;
  }
  // one thread per (head, pair): every load of a token is in flight at once
  const int work = max((q_heads + kv_heads) * d / 2, kv_heads * d);
  const int threads = work >= 256 ? 256 : (work >= 128 ? 128 : 64);
  const dim3 grid(tokens, min(64, (work + threads - 1) / threads));
  LRM_LAUNCH(rope_store_kernel<A>, grid, threads, 0, stream, static_cast<const A*>(qkv),
             static_cast<A*>(q_out), static_cast<A*>(k_out), static_cast<A*>(v_out),
             static_cast<A*>(k_pages), static_cast<A*>(v_pages), dest_rows, positions, inv_freq,
             rotary, q_heads, kv_heads, d, page_size);
  return 0;
}

LRM_API int lrm_rope_store(const void* qkv, int dtype, void* q_out, void* k_out, void* v_out,
                           void* k_pages, void* v_pages, const int* dest_rows,
                           const int* positions, const float* inv_freq, int rotary, int tokens, int q_heads,
                           int kv_heads, int d, int page_size, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (d <= 0 || d % 2 != 0 || rotary < 0 || rotary > d || rotary % 2 != 0 || q_heads <= 0 ||
      kv_heads < 0 || page_size <= 0)
    return LRM_BAD_ARGUMENT;
  if ((k_pages == nullptr) != (v_pages == nullptr)) return LRM_BAD_ARGUMENT;
  if (k_pages != nullptr && dest_rows == nullptr) return LRM_BAD_ARGUMENT;
  if (dtype == LRM_F32)
    return launch_rope<float>(qkv, q_out, k_out, v_out, k_pages, v_pages, dest_rows, positions, inv_freq,
                              rotary, tokens, q_heads, kv_heads, d, page_size, stream);
  if (dtype == LRM_BF16)
    return launch_rope<__nv_bfloat16>(qkv, q_out, k_out, v_out, k_pages, v_pages, dest_rows, positions,
                                      inv_freq, rotary, tokens, q_heads, kv_heads, d, page_size, stream);
  return LRM_BAD_ARGUMENT;
}

// (cos, sin) of float(position) * inv_freq[i] for every token of a step and i < half: the table
// that a product's rotating epilogue reads, the same angles and the same sincosf as above.
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                  float2* __restrict__ table, int tokens, int half) {
  pdl_trigger();
  pdl_wait();
  const int item = blockIdx.x * blockDim.x + threadIdx.x;
  if (item >= tokens * half) return;
  const float angle = __fmul_rn(static_cast<float>(positions[item / half]), inv_freq[item % half]);
  float sn, cs;
  sincosf(angle, &sn, &cs);
  table[item] = make_float2(cs, sn);
}

LRM_API int lrm_rope_table(const int* positions, const float* inv_freq, float* table, int tokens, int half,
                           cudaStream_t stream) {
  if (tokens <= 0 || half <= 0) return 0;
  const int items = tokens * half;
  LRM_LAUNCH(rope_table_kernel, dim3((items + 255) / 256), 256, 0, stream, positions, inv_freq,
             reinterpret_cast<float2*>(table), tokens, half);
  return 0;
}
