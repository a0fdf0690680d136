// Entry points for callers that may not allocate device memory.
//
// This header has no counterpart in the reference engine: it exists for embedders of this
// library that run where cudaMalloc is off limits, for instance inside a host application
// that hands out all device memory itself at start-up, in a real-time loop where an
// allocation could stall on the driver, or after memory has been handed over completely to
// other pools so that a late allocation could fail.  Such callers own their inputs and
// outputs; what they cannot provide is the scratch a kernel needs between its two passes.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Size of the scratch that every no-allocation entry point shares on a device.  It is part
// of the library image: each GPU that loads the library holds this much until exit.
#define INFERO_STATIC_SCRATCH_BYTES (4ll << 20)

// Decode attention over the paged cache (the same arguments and result as infero_attn_decode,
// without its scratch pointer): the partial results of the context splits go to a fixed
// array inside the library instead of memory the caller allocates.
//
//   * Nothing is allocated, by cudaMalloc or otherwise; on the first call on a device the
//     library looks up the array's device address (cudaGetSymbolAddress) and keeps it.
//     Make that first call before any stream capture starts on the device.
//   * n_tok * n_heads * n_splits * (head_dim + 2) * 4 bytes must fit in
//     INFERO_STATIC_SCRATCH_BYTES; a larger request is refused with an error (returns
//     non-zero, see infero_last_error) and launches nothing.
//   * Every call on a device uses the same array and finds the previous call's contents in
//     it.  The kernels write each partial result before they read it, so nothing needs to
//     be cleared; but two calls whose kernels overlap on the GPU (different streams without
//     an ordering between them) race on the array.  Keep them on one stream or order them.
int infero_attn_decode_static(const void* q, int q_stride, void* out, int out_stride, const void* k_cache,
                              const void* v_cache, const int* block_table, int max_blocks, const int* tok_entry,
                              const int* positions, int tok_first, int n_tok, int n_heads, int n_kv, int head_dim,
                              int page_size, int window, float scale, int chunk, int n_splits,
                              cudaStream_t stream);

#ifdef __cplusplus
}
#endif
