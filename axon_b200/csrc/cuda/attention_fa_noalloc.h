// Split-key decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference implementation; it exists for
// users of this library.
//
// Who needs it: code that runs where cudaMalloc is off limits.  Examples are a host
// program that hands this library a fixed set of buffers it carved out of its own
// arena at start-up and forbids any later allocation (so that its memory plan stays
// exact and a step can never fail half-way with an out-of-memory error), a plug-in
// loaded into a process whose allocator the plug-in must not bypass, and a caller in
// the middle of work during which the CUDA runtime refuses allocations.  The regular
// entry point (axon_attention_fa) needs scratch memory for the partial results of the
// key splits and expects the caller to allocate it; this one brings its own.
//
// How: the scratch lives in a file-scope `static __device__` array of
// AXON_FA_NOALLOC_SCRATCH_FLOATS floats (16 MiB) inside libaxon_cuda.so.  Every GPU
// on which the library is loaded holds that array until the process exits.  The
// function calls no cudaMalloc, cudaFree or any other allocating routine.
//
// Limits and rules:
//  * n_items * kv_heads * n_splits * 16 * (head_dim + 2) must not exceed
//    AXON_FA_NOALLOC_SCRATCH_FLOATS; a larger launch is refused with a message
//    (axon_last_error) and nothing runs.  With head size 128 and 4 kv heads that is,
//    for instance, 64 requests with up to 8 splits each.
//  * The first call on a device looks up the array's device address
//    (cudaGetSymbolAddress) and remembers it.  Make that first call outside of any
//    stream capture.
//  * All calls share the one array, which keeps whatever the last call left in it.
//    Nothing in it has to start at zero: every slot a launch reads was written by the
//    same launch before.  Two calls whose kernels may overlap on the GPU (different
//    streams without an ordering between them) race on the array; order them.
//
// Arguments are those of axon_attention_fa with `decode` fixed to 1 and without the
// scratch pointer; inputs and outputs are still the caller's.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "kv_layout.h"   // struct AxonKvLayout, the cache description a caller fills in

#define AXON_FA_NOALLOC_SCRATCH_FLOATS (4ll * 1024 * 1024)
// arrival counters of the key splits, one per (item, kv head); launches with more items fold
// their splits in a second kernel instead
#define AXON_FA_NOALLOC_COUNTERS 4096

#ifdef __cplusplus
extern "C" {
#endif

// Returns 0 on success, 1 when the arguments are refused, 2 when a CUDA call failed.
__attribute__((visibility("default")))
int axon_attention_fa_decode_noalloc(const void* q, const void* pool, void* out, const int32_t* segments,
                                     int n_segments, const int32_t* items, int n_items,
                                     const struct AxonKvLayout* layout, int heads, float scale, int window,
                                     int tokens_per_tile, int n_splits, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
