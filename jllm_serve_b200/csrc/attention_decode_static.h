// jllm_attention_decode_static: paged decode attention that asks the caller for no scratch memory.
//
// This entry point has no counterpart in beniaminp/jllm-serve; it exists for users of this library.
//
// Who it is for. jllm_attention_decode splits a long key range over several thread blocks and needs
// scratch memory for their partial results, which its caller has to allocate. Some callers cannot: a
// serving process that handed the whole GPU to its cache pool at start-up and has nothing left to
// carve from; a host program that owns all device memory itself and forbids library-side allocation;
// a decode loop that must not meet the device-wide synchronisation that cudaMalloc and cudaFree imply.
// For them the scratch lives inside the library, in a file-scope device array of fixed size.
//
// What to know.
//  * Limit: rows * heads * splits * (head_dim + 2) floats must fit JLLM_ATTENTION_DECODE_STATIC_FLOATS
//    (2 Mi floats = 8 MiB). Larger requests are refused with an error that says so; nothing is launched.
//    With one split no scratch is used at all.
//  * Cost: every GPU on which the library is loaded holds the 8 MiB from load until the process exits.
//  * Set-up: the first call on a device looks up the array's device address (cudaGetSymbolAddress, with
//    that device current) and remembers it. Make that first call before any stream capture begins.
//  * No allocation: the call performs no cudaMalloc, cudaFree or other allocating routine; inputs and
//    outputs are the caller's, as for jllm_attention_decode, whose kernels and results it shares.
//  * One array for all calls: it keeps the last call's partial results and every call overwrites what it
//    reads, so nothing needs clearing, but two calls that overlap on the GPU (different streams, or
//    different host threads without ordering) race on it. Order them on one stream, or use
//    jllm_attention_decode with separate scratch.
#pragma once

#include <cuda_runtime.h>

#define JLLM_ATTENTION_DECODE_STATIC_FLOATS (2 * 1024 * 1024)

#ifdef __cplusplus
extern "C" {
#endif

// Arguments as jllm_attention_decode without the scratch pointer. Returns 0, or an error code whose text
// jllm_last_error() gives.
int jllm_attention_decode_static(const void* q, int q_stride, const void* k_cache, const void* v_cache, void* out,
                                 int out_stride, const int* row_seg, const int* row_pos, const int* block_tables,
                                 int table_stride, int rows, int heads, int kv_heads, int head_dim, int page_size,
                                 int window, float scale, int splits, cudaStream_t stream);

// The capacity of the built-in scratch in floats.
long long jllm_attention_decode_static_capacity(void);

#ifdef __cplusplus
}
#endif
