// Shared by the kernels that choose a token: the order among candidates (ties go to the lower
// id), the counter-based noise of temperature sampling, and the host entry of the reduction over
// per-piece results.
#pragma once
#include "common.cuh"

__device__ __forceinline__ uint64_t mix64(uint64_t z) {
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  return z ^ (z >> 31);
}

// uniform in (0,1) with 24 random bits, exactly representable in float32
__device__ __forceinline__ float hash_uniform(uint64_t seed, uint64_t key, uint32_t i) {
  const uint64_t z = mix64(mix64(seed + 0x9e3779b97f4a7c15ull * (key + 1)) + i);
  return (static_cast<float>(static_cast<uint32_t>(z >> 40)) + 0.5f) * (1.0f / 16777216.0f);
}

struct Best {
  float value;
  int id;
};
__device__ __forceinline__ Best better(Best a, Best b) {
  // ids < 0 mean "nothing"; a non-finite value never wins because its row is rejected anyway
  if (b.id >= 0 && (a.id < 0 || b.value > a.value || (b.value == a.value && b.id < a.id))) return b;
  return a;
}

// -log(-log u) with u from the hash of (seed, key, i): the Gumbel noise added to logit i / T.
__device__ __forceinline__ float gumbel_noise(uint64_t seed, uint64_t key, uint32_t i) {
  return -logf(-logf(hash_uniform(seed, key, i)));
}

// A candidate as one 64-bit word whose unsigned order is the order of better(): the score's bits
// made monotonic (sign flipped, negatives inverted) above the id counted down, so that among equal
// scores the lower id is the larger word. 0 is below every candidate. Scores must not be NaN.
__device__ __forceinline__ unsigned long long pick_key(float value, int id) {
  const uint32_t bits = __float_as_uint(value + 0.0f);  // -0 and +0 are one score
  const uint32_t ordered = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
  return (static_cast<unsigned long long>(ordered) << 32) | (0xffffffffu - static_cast<uint32_t>(id));
}
__device__ __forceinline__ int pick_key_id(unsigned long long key) {
  return key == 0ull ? -1 : static_cast<int>(0xffffffffu - static_cast<uint32_t>(key & 0xffffffffull));
}

// out[row] = id of the best of `pieces` (value, id) candidates per row, -1 when a piece is marked -2
// (it saw a non-finite logit). Defined in sampling.cu.
extern "C" int lrm_pick_reduce(const float* piece_value, const int* piece_id, int* out, int rows, int pieces,
                               cudaStream_t stream);
// out[row] = id of the row's winning pick_key in best[row], or -1 when bad[row] is set or nothing
// was offered; both arrays are zero again afterwards. Defined in sampling.cu.
extern "C" int lrm_pick_winners(unsigned long long* best, int* bad, int* out, int rows, cudaStream_t stream);
