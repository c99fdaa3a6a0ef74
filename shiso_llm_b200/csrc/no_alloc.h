// Decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference; it exists for embedders of this
// library, not for the engine (which allocates its scratch through PyTorch's caching
// allocator and never calls this).
//
// Who needs it.  Two kinds of caller cannot hand the split-key decode attention the scratch
// buffer it normally asks for: a host program that has given all device memory to a pool of
// its own and forbids (or simply has no room for) any further cudaMalloc; and a caller on a
// latency-critical path, for whom the device-wide synchronisation that cudaMalloc and
// cudaFree imply is not acceptable.  For them the partial results of the key ranges live in
// a fixed array inside the library's device image instead.
//
// What it costs.  The array is SHISO_NO_ALLOC_SCRATCH_FLOATS floats (4 MiB).  Every GPU on
// which this library's device code is loaded holds that memory until the process exits,
// whether or not this function is ever called.
//
// Limits and rules.
//  * The scratch needed is tokens * heads * splits * (head_dim + 2) floats; a call that needs
//    more than the array holds is refused with SHISO_ERR_TOO_LARGE and nothing is launched.
//    shiso_no_alloc_last_error() then returns a sentence with both numbers.
//  * The caller passes inputs and outputs as for shiso_decode_attention; only the scratch
//    argument is gone.  The function calls no cudaMalloc, cudaFree or allocating library
//    routine.
//  * The first call on a device looks up the array's device address
//    (cudaGetSymbolAddress, with that device current) and keeps it; make that first call
//    before any stream capture begins on that device.
//  * All calls share the one array, and it keeps the previous call's contents.  Nothing in it
//    has to start at zero: every slot a call reads is written by that call first (a key range
//    that is empty writes "no keys" into its slot).  Two calls that overlap on the GPU - on
//    different streams, or from different threads - race on the array; run them one after
//    the other on one stream, or order them with events.
#pragma once

#include <cuda_runtime.h>

#define SHISO_NO_ALLOC_SCRATCH_FLOATS (1 << 20)
#define SHISO_ERR_TOO_LARGE 1005

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments and result as shiso_decode_attention without the scratch pointer.
// Returns 0, a SHISO_ERR_* code, or a cudaError_t value.
__attribute__((visibility("default"))) int shiso_decode_attention_no_alloc(
    const void* q, const void* k_cache, const void* v_cache, const int* block_table, int table_width,
    const int* positions, const int* seq_of_token, void* out, int tokens, int heads, int kv_heads, int head_dim,
    int page_size, float scale, int window, int splits, cudaStream_t stream);

// The reason for the last refusal on the calling thread ("" when there was none).
__attribute__((visibility("default"))) const char* shiso_no_alloc_last_error(void);

#ifdef __cplusplus
}
#endif
