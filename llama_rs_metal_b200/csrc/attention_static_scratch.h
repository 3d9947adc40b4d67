// Decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference (which allocates its
// split-attention partials from a per-session workspace); it exists for hosts
// of this library that cannot call cudaMalloc or any allocator at the time
// they run a step: code inside a real-time or fault-handling path that is not
// allowed to block on the driver's allocator, plugins running under a host
// process that owns all device memory, and launches issued while another
// thread holds a lock the allocator would need.
//
// It computes exactly what lrm_attention_decode_tiled computes (one query per
// sequence over the paged bfloat16 cache, split over the keys, partials merged
// in split order) but keeps the partials in a file-scope __device__ array of
// lrm_attention_static_scratch_floats() floats (4 MiB) that every device which
// loads the library holds until the process exits. The caller still passes all
// inputs and the output.
//
//  * Nothing is allocated or freed, by this function or by anything it calls.
//  * A problem whose partials (seqs * q_heads * n_splits * (head_dim + 2) floats)
//    do not fit is refused with LRM_SCRATCH_EXCEEDED; choose fewer splits.
//  * The first call on each device looks the array's device address up
//    (cudaGetSymbolAddress, with that device current) and remembers it. Make
//    that first call outside any stream capture.
//  * All calls on a device share the one array, and it keeps whatever the last
//    call left there. Nothing in it has to start at zero: every call writes
//    each partial it later reads. Two calls that overlap on the GPU (different
//    streams, or graphs replayed concurrently) race on it; run them one after
//    another.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { LRM_SCRATCH_EXCEEDED = -4 };

// Capacity of the static scratch array, in floats.
int lrm_attention_static_scratch_floats(void);

// 0 on success; LRM_SCRATCH_EXCEEDED, -1 (bad argument), -2 (unsupported size) or a
// positive cudaError_t otherwise. Arguments as lrm_attention_decode_tiled, minus the scratch.
int lrm_attention_decode_tiled_static_scratch(const void* q, const void* k_pages, const void* v_pages,
                                              void* out, const int* page_table, int table_stride,
                                              const int* slots, const int* kv_lens, int seqs,
                                              int q_heads, int kv_heads, int head_dim, int page_size,
                                              float scale, int window, int n_splits,
                                              cudaStream_t stream);

// A sentence for each code the function above returns.
const char* lrm_attention_static_scratch_error(int code);

#ifdef __cplusplus
}
#endif
