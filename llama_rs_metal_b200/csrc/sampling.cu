// Token choice on the device over rows of float32 logits, in two small stages so that a
// long row is scanned by many blocks.
//
// Greedy: the largest logit, lowest id on ties; a row with any non-finite
// logit yields -1 (reference: crates/metal-backend/src/shaders/sampling.metal:39-80,
// whose sentinel is 0xffffffff).
//
// Temperature: Gumbel-max. id = argmax_i( logit_i / T + g_i ), g_i =
// -log(-log u_i), u_i from a counter-based hash of (seed, key, i). `key` is
// given per row by the caller (it encodes request and step), so a row's choice
// does not depend on what else is in the batch, and no ordered prefix sum over
// the vocabulary is needed. The draw is distributed as softmax(logits / T).
#include "common.cuh"
#include "pick.cuh"

// Stage 1: block (row, piece) scans its piece of the row and leaves its best (value, id) and
// whether it saw a non-finite logit. Stage 2: one block per row reduces the pieces.
// Ties always go to the lower id, so the result does not depend on how a row is cut.
template <bool GUMBEL>
__global__ void pick_pieces_kernel(const float* __restrict__ logits, float* __restrict__ piece_value,
                                   int* __restrict__ piece_id, int vocab, int piece,
                                   float inv_temperature, uint64_t seed,
                                   const long long* __restrict__ keys) {
  __shared__ float s_value[32];
  __shared__ int s_id[32];
  __shared__ int s_bad;
  pdl_trigger();  // let the next kernel be scheduled; it waits for this one where it must
  pdl_wait();
  const int row = blockIdx.y;
  const float* x = logits + static_cast<size_t>(row) * vocab;
  const uint64_t key = GUMBEL ? static_cast<uint64_t>(keys[row]) : 0ull;
  if (threadIdx.x == 0) s_bad = 0;
  __syncthreads();
  Best best{-INFINITY, -1};
  bool bad = false;
  const int begin = blockIdx.x * piece, end = min(vocab, begin + piece);
  for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
    float v = x[i];
    bad |= !isfinite(v);
    if (GUMBEL) {
      v = fmaf(v, inv_temperature, gumbel_noise(seed, key, static_cast<uint32_t>(i)));
    }
    best = better(best, Best{v, i});
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best other{__shfl_xor_sync(0xffffffffu, best.value, o), __shfl_xor_sync(0xffffffffu, best.id, o)};
    best = better(best, other);
  }
  if (bad) atomicOr(&s_bad, 1);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    s_value[warp] = best.value;
    s_id[warp] = best.id;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    Best total{-INFINITY, -1};
    for (int w = 0; w < (blockDim.x + 31) / 32; ++w) total = better(total, Best{s_value[w], s_id[w]});
    const size_t o = static_cast<size_t>(row) * gridDim.x + blockIdx.x;
    piece_value[o] = total.value;
    piece_id[o] = s_bad ? -2 : total.id;  // -2: this piece saw a non-finite logit
  }
}

__global__ void pick_reduce_kernel(const float* __restrict__ piece_value,
                                   const int* __restrict__ piece_id, int* __restrict__ out,
                                   int pieces) {
  __shared__ float s_value[32];
  __shared__ int s_id[32];
  __shared__ int s_bad[32];
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  Best best{-INFINITY, -1};
  bool bad = false;
  for (int i = threadIdx.x; i < pieces; i += blockDim.x) {
    const int id = piece_id[static_cast<size_t>(row) * pieces + i];
    bad |= id == -2;
    best = better(best, Best{piece_value[static_cast<size_t>(row) * pieces + i], id});
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best other{__shfl_xor_sync(0xffffffffu, best.value, o), __shfl_xor_sync(0xffffffffu, best.id, o)};
    best = better(best, other);
  }
  bad = __any_sync(0xffffffffu, bad);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
  if (warps == 1) {
    if (threadIdx.x == 0) out[row] = bad ? -1 : best.id;
    return;
  }
  if (lane == 0) {
    s_value[warp] = best.value;
    s_id[warp] = best.id;
    s_bad[warp] = bad;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    Best total{-INFINITY, -1};
    bool any_bad = false;
    for (int w = 0; w < warps; ++w) {
      total = better(total, Best{s_value[w], s_id[w]});
      any_bad |= s_bad[w] != 0;
    }
    out[row] = any_bad ? -1 : total.id;
  }
}

constexpr int kPiece = 4096;  // logits one stage-1 block scans

// The second stage alone (also the end of the head product that chooses in its epilogue): a warp
// per row for a few pieces, a block of 256 threads for thousands.
LRM_API int lrm_pick_reduce(const float* piece_value, const int* piece_id, int* out, int rows, int pieces,
                            cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (pieces <= 0 || piece_value == nullptr || piece_id == nullptr || out == nullptr) return LRM_BAD_ARGUMENT;
  LRM_LAUNCH(pick_reduce_kernel, dim3(rows), pieces > 256 ? 256 : 32, 0, stream, piece_value, piece_id, out, pieces);
  return 0;
}

// scratch: rows * pieces floats and as many ints, pieces = ceil(vocab / 4096)
LRM_API int lrm_pick_pieces(int vocab) { return (vocab + kPiece - 1) / kPiece; }

// The end of a head product that chose in its epilogue (csrc/gemm_bf16_stream.cu, epilogue 5).
__global__ void pick_winners_kernel(unsigned long long* __restrict__ best, int* __restrict__ bad,
                                    int* __restrict__ out, int rows) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= rows) return;
  const unsigned long long key = best[row];
  const int flag = bad[row];
  out[row] = flag ? -1 : pick_key_id(key);
  best[row] = 0ull;  // ready for the next product
  bad[row] = 0;
}

LRM_API int lrm_pick_winners(unsigned long long* best, int* bad, int* out, int rows, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (best == nullptr || bad == nullptr || out == nullptr) return LRM_BAD_ARGUMENT;
  LRM_LAUNCH(pick_winners_kernel, dim3((rows + 63) / 64), 64, 0, stream, best, bad, out, rows);
  return 0;
}

static int pick_rows(const float* logits, int* out, float* piece_value, int* piece_id, int rows,
                     int vocab, bool gumbel, float inv_temperature, uint64_t seed,
                     const long long* keys, cudaStream_t stream) {
  const int pieces = lrm_pick_pieces(vocab);
  if (rows > 65535) return LRM_UNSUPPORTED;
  const dim3 grid(pieces, rows);
  if (gumbel)
    LRM_LAUNCH(pick_pieces_kernel<true>, grid, 256, 0, stream, logits, piece_value, piece_id, vocab, kPiece,
               inv_temperature, seed, keys);
  else
    LRM_LAUNCH(pick_pieces_kernel<false>, grid, 256, 0, stream, logits, piece_value, piece_id, vocab, kPiece,
               1.f, static_cast<uint64_t>(0), static_cast<const long long*>(nullptr));
  return lrm_pick_reduce(piece_value, piece_id, out, rows, pieces, stream);
}

LRM_API int lrm_argmax_rows(const float* logits, int* out, float* piece_value, int* piece_id,
                            int rows, int vocab, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0 || piece_value == nullptr || piece_id == nullptr) return LRM_BAD_ARGUMENT;
  return pick_rows(logits, out, piece_value, piece_id, rows, vocab, false, 1.f, 0ull, nullptr, stream);
}

LRM_API int lrm_sample_gumbel_rows(const float* logits, int* out, float* piece_value, int* piece_id,
                                   int rows, int vocab, float temperature, unsigned long long seed,
                                   const long long* keys, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0 || !(temperature > 0.f) || keys == nullptr || piece_value == nullptr ||
      piece_id == nullptr)
    return LRM_BAD_ARGUMENT;
  return pick_rows(logits, out, piece_value, piece_id, rows, vocab, true, 1.0f / temperature, seed,
                   keys, stream);
}
