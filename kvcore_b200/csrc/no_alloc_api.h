// Split-KV paged attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference project; it exists for hosts that
// embed this library under a fixed memory plan.  Two kinds of caller are meant:
//
//  * programs that carve up the GPU's memory themselves at start-up (an inference server
//    that gives each engine a hard partition, a real-time pipeline with a certified memory
//    map) and therefore forbid the libraries they load from calling cudaMalloc at all;
//  * code on a latency-critical path, where cudaMalloc and cudaFree are off limits because
//    they synchronise the whole device and stall every other stream.
//
// The regular entry point (kvb_flash_paged_attention) takes its split-KV scratch from the
// caller, who normally gets it from an allocator.  This variant keeps the scratch, and the
// status word, in a fixed array inside the library image instead.  What that means for you:
//
//  * The array is KVB_STATIC_SCRATCH_FLOATS floats (8 MiB).  Every GPU that loads the
//    library holds it until the process exits, used or not.
//  * A call needs  num_reqs * KVH * num_splits * 16 * (D + 2)  floats when num_splits > 1.
//    A call that needs more is refused with an error (nothing is launched).
//  * The first call on each device looks up the array's device address
//    (cudaGetSymbolAddress).  Make that first call during start-up, with the device
//    current, and before any stream capture.
//  * All calls share the one array, and it keeps whatever the last call left in it.  The
//    kernels write every partial result they later read, so nothing has to be cleared
//    between calls.  The status word beside it starts at zero when the library is loaded
//    and only ever gains bits: a problem reported by one call is still there after any
//    number of later calls, until kvb_static_status reads and clears it.
//    Two calls that overlap on the GPU (different streams, no dependency between them)
//    race on the array: keep calls on one stream, or order them with events.
//  * num_splits is at most 1024.
//  * It calls no cudaMalloc, cudaFree, or allocating library routine; inputs and outputs
//    are the caller's buffers.
//
// Arguments are those of kvb_flash_paged_attention without the scratch pointer: bf16 q, K/V
// caches [pages, KVH, page_size, D], int32 block table, query_start [num_reqs + 1] and
// context_lens [num_reqs] on the device.  Decode shape only when num_splits > 1:
// max_query_len * (H / KVH) <= 16.  Returns 0, or a negative code with the message available
// from kvb_last_error().  kvb_static_status reads (and clears) the status bits that all calls
// since its last use have set on the current device (2: a page id outside the cache); it
// synchronises the device.
#pragma once

#include <cuda_runtime.h>

#define KVB_STATIC_SCRATCH_FLOATS (2 * 1024 * 1024)

#ifdef __cplusplus
extern "C" {
#endif

int kvb_flash_paged_attention_static(void* out, long long out_stride, const void* q, long long q_stride,
                                     const void* k_cache, const void* v_cache, const int* table,
                                     int table_stride, const int* query_start, const int* context_lens,
                                     int num_reqs, int max_query_len, int H, int KVH, int D, int page_size,
                                     int num_pages, float scale, int window, int num_splits,
                                     cudaStream_t stream);

int kvb_static_status(int* out);

#ifdef __cplusplus
}
#endif
