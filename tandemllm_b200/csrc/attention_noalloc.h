// An entry point of the split attention kernel for callers that cannot allocate device memory.
//
// It has no counterpart in the reference project: this engine adds it for programs that use the kernel library
// directly, without the Python engine around it.
//
// Who cannot allocate, and why. The split attention kernel needs scratch memory for its per-span partial results, and
// the ordinary entry point (tl_paged_attention_split) leaves it to the caller to bring that memory. Some callers have
// nowhere to get it from: a serving loop that must not call cudaMalloc or cudaFree because both may synchronise the
// whole device and stall every stream; a process that handed all device memory to another allocator at start-up, so
// that a later cudaMalloc simply fails; a host program in another language that links this library for one kernel and
// has no device allocator of its own. For them the scratch lives inside the library, in a fixed array in device memory.
//
// What the fixed array costs and limits. The array holds TL_STATIC_SCRATCH_FLOATS 32-bit floats (8 MiB). Every GPU on
// which the library is loaded keeps that much memory from the moment the library is loaded until the process exits,
// whether or not this entry point is ever called. A call needs rows * Hq * n_spans * (D + 2) floats (what
// tl_attention_scratch_floats returns); a call that needs more than the array holds is refused with a message and
// launches nothing. 8 MiB covers, for example, 8 rows of 32 heads of size 64 over 128 spans (contexts of 32,768).
//
// Rules for callers.
//  * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with that device current)
//    and keeps it. Make that first call outside any stream capture.
//  * Every call on a device shares the one array. Calls whose kernels may run at the same time on that device (two
//    streams, two host threads) race on it and give wrong results; run them one after another on one stream.
//  * Nothing in the array has to start at zero and nothing is cleared: the join kernel reads exactly the elements that
//    the span kernel of the same call wrote. What an earlier call left behind is never read.
//  * `n_spans` must cover the longest row: n_spans >= max(positions) / 256 + 1 (what tl_attention_spans returns for the
//    longest context). A row that lies past it is not read out of bounds: its keys beyond the last span are left out, the
//    status word gets 3, and the result of that row is wrong. `num_pages` is the number of pages in k_cache and v_cache;
//    a block-table entry at or beyond it is treated as a missing page (status 3), as everywhere in this library
//    (0: the pool's size is unknown and only an entry's sign is checked).
//  * It calls no cudaMalloc, no cudaFree and no library routine that allocates. Inputs, outputs, the block table and
//    the status word are the caller's, exactly as for tl_paged_attention_split.
#pragma once

#include <cuda_runtime.h>

#define TL_STATIC_SCRATCH_FLOATS (2 * 1024 * 1024)

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments and result as tl_paged_attention_split without its `scratch` argument. Returns 0, a cudaError_t, or
// TL_BAD_ARGUMENT (100001) after storing a message that tl_last_error() returns.
int tl_paged_attention_split_static(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                                    int max_pages, int page_size, int num_pages, const int* req_of_row, const int* positions,
                                    float scale, int window, void* out, int rows, int Hq, int Hk, int D, int n_spans,
                                    int dtype, int* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
