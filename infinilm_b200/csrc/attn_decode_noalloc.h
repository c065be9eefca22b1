// Decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in InfiniLM; it is an addition of this package.
//
// Who needs it: code that runs where cudaMalloc is off limits - a host thread inside a region
// where the allocator must not be entered (a real-time loop, a signal-safe section, a plugin
// whose host forbids allocation after start-up), or an application that has handed all device
// memory to its own pool and gives a library no way to ask for more. The regular entry point,
// il_attn_decode, expects the caller to bring two scratch buffers sized by the batch and the
// number of key splits; such a caller has nowhere to get them from. Here the scratch lives in a
// fixed array inside the library's device image instead, so the call needs inputs and outputs only.
//
// The price, and the rules:
//  * The array holds IL_NOALLOC_MAX_ROWS * (HEAD_DIM + 2) floats (about 4.2 MB at head_dim 128).
//    Every GPU that loads the library carries it until the process exits.
//  * n_decode * n_heads * n_splits must not exceed IL_NOALLOC_MAX_ROWS; a larger call is refused
//    with IL_NOALLOC_TOO_LARGE and nothing is launched.
//  * The first call on a device looks up the array's device address (cudaGetSymbolAddress with that
//    device current) and remembers it. That lookup is not a stream operation: make the first call
//    on each device before any stream capture begins. Nothing locks that lookup: two host threads that
//    make their first call on one device at the same moment both ask the runtime and both store the
//    same address, which is harmless.
//  * All calls share the one array. It keeps whatever the last call left there; the kernels write
//    every partial result before they read it, so nothing has to be cleared between calls. Two
//    calls that overlap on the GPU (different streams, no ordering between them) race on it.
//  * No cudaMalloc, cudaFree or allocating library routine is called, on any call.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define IL_NOALLOC_MAX_ROWS 8192
#define IL_NOALLOC_TOO_LARGE (-3)
#define IL_NOALLOC_NO_SYMBOL (-4)

// Same arguments as il_attn_decode without the two scratch pointers. Returns 0 when both kernels
// were launched, IL_NOALLOC_TOO_LARGE when the call needs more scratch than the array holds,
// IL_NOALLOC_NO_SYMBOL when the array's address could not be obtained, a negative argument code,
// or 1000 + cudaError_t of a failed launch.
int il_attn_decode_noalloc(const void* qkv, int row_stride, void* out, const void* cache, const int* block_table,
                           int bt_stride, const int* entry_kvlen, int page_size, int n_decode, int nh, int nkv, int hd,
                           float scale, int window, int pages_per_split, int n_splits, cudaStream_t stream);

// A sentence for each code this entry point returns.
const char* il_attn_decode_noalloc_strerror(int code);

// Rows of scratch (n_decode * n_heads * n_splits) the array can hold, and its size in bytes.
int il_attn_decode_noalloc_max_rows(void);
long long il_attn_decode_noalloc_scratch_bytes(void);

#ifdef __cplusplus
}
#endif
