// Token embedding: hidden[t,:] = table[ids[t],:] * scale, widened to the float32
// residual stream (scale 1 is exact, so a model without an embedding scale pays nothing).
// An id outside the table writes zeros; the host rejects such
// ids before launch (reference: crates/metal-backend/src/shaders/matrix.metal:94-103).
#include "common.cuh"

int g_lrm_pdl = 1;

// Switch programmatic dependent launch on or off for every kernel of the library.
LRM_API void lrm_set_pdl(int enabled) { g_lrm_pdl = enabled ? 1 : 0; }

template <typename W>
__global__ void embed_rows_kernel(const W* __restrict__ table, const int* __restrict__ ids,
                                  float* __restrict__ out, int hidden, int vocab, float scale) {
  pdl_trigger();  // a small kernel: let the next one start (and prefetch its weights) right away
  pdl_wait();
  const int t = blockIdx.x;
  const int id = ids[t];
  const bool ok = id >= 0 && id < vocab;
  const W* row = table + static_cast<size_t>(ok ? id : 0) * hidden;
  float* dst = out + static_cast<size_t>(t) * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = ok ? to_f32(row[i]) * scale : 0.f;
}

LRM_API int lrm_embed_rows(const void* table, int table_dtype, const int* ids, float* out,
                           int tokens, int hidden, int vocab, float scale, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (hidden <= 0 || vocab <= 0) return LRM_BAD_ARGUMENT;
  const int threads = hidden >= 256 ? 256 : 64;
  if (table_dtype == LRM_F32)
    LRM_LAUNCH(embed_rows_kernel<float>, tokens, threads, 0, stream, static_cast<const float*>(table), ids, out,
               hidden, vocab, scale);
  else if (table_dtype == LRM_BF16)
    LRM_LAUNCH(embed_rows_kernel<__nv_bfloat16>, tokens, threads, 0, stream,
               static_cast<const __nv_bfloat16*>(table), ids, out, hidden, vocab, scale);
  else
    return LRM_BAD_ARGUMENT;
  LRM_LAUNCH_CHECK();
  return 0;
}
