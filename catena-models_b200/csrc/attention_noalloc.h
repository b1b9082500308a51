// Decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in catena-models; it exists for embedders of this
// library that cannot call cudaMalloc themselves and cannot let a library do it for them:
// code running inside a captured region or under a strict memory budget set by its host
// application, plugins loaded into a process whose allocator is owned by someone else, and
// C callers that have no torch allocator to ask for the kernel's scratch buffers.
//
// cm_attn_decode_noalloc() computes exactly what cm_attn_decode() computes (attention.cu:
// decode attention of one new token per sequence over the paged cache, split over fixed
// chunks of cache entries and merged in chunk order).  The difference is where the per-chunk
// partial results live: instead of two caller-provided scratch buffers they are kept in one
// array that is part of the library image itself.
//
//   * Limit: the array holds CM_NOALLOC_SCRATCH_FLOATS floats (5 MiB).  It is resident on every
//     GPU that loads the library, from load until the process exits.  A call needs
//     B * QH * n_chunks * (HD + 2) floats; a call that needs more is refused with CM_ERR_SHAPE
//     and a message (cm_last_error), nothing is launched.
//   * The first call on each device looks up the array's device address (once per device, with
//     that device current).  Make that first call outside of any stream capture.
//   * No call allocates or frees: no cudaMalloc, cudaFree, or allocating library routine.
//   * All calls share the one array and it keeps whatever the last call left in it.  The
//     kernels write every partial result before they read it, so nothing has to be cleared
//     between calls; but two calls whose kernels overlap on the GPU (different streams, no
//     ordering between them) would overwrite each other's partial results.  Order such calls.
#pragma once
#include <cuda_runtime.h>

#define CM_NOALLOC_SCRATCH_FLOATS (5 * 256 * 1024)

#ifdef __cplusplus
extern "C" {
#endif

// Arguments as cm_attn_decode, without the two scratch pointers.  Returns 0, or a negative
// code with the reason in cm_last_error().
int cm_attn_decode_noalloc(int dt, void* ctx, long long ldc, const void* q, long long ldq, const void* gate,
                           long long ldg, const int* seq_pos, const int* seq_slot, const void* pool,
                           long long pages, const int* ptab, int ptab_stride, int ring, int window, int B,
                           int QH, int KVH, int HD, int n_chunks, float scale, cudaStream_t st);

#ifdef __cplusplus
}
#endif
