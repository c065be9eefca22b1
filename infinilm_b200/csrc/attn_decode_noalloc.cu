// il_attn_decode_noalloc: the split-KV decode attention of attn_decode.cu with its scratch in a
// file-scope device array, for callers that cannot allocate (see attn_decode_noalloc.h).
// The kernels are those of attn_decode.cu, compiled into this library a second time.
#include "attn_decode.cu"
#include "attn_decode_noalloc.h"

// Partials of all splits: IL_NOALLOC_MAX_ROWS rows of head_dim floats, then the (max, sum) pairs.
static __device__ __align__(256) float il_noalloc_scratch[(size_t)IL_NOALLOC_MAX_ROWS * (HEAD_DIM + 2)];

#define IL_NOALLOC_MAX_DEVICES 64
static float* il_noalloc_addr[IL_NOALLOC_MAX_DEVICES];    // device address of the array, per device (0: not looked up)

extern "C" __attribute__((visibility("default")))
int il_attn_decode_noalloc(const void* qkv, int row_stride, void* out, const void* cache, const int* block_table,
                           int bt_stride, const int* entry_kvlen, int page_size, int n_decode, int nh, int nkv, int hd,
                           float scale, int window, int pages_per_split, int n_splits, cudaStream_t stream) {
    if (n_decode <= 0) return IL_OK;
    if (hd != HEAD_DIM || page_size != AD_PAGE) return IL_UNSUPPORTED;
    if (nh <= 0 || nkv <= 0 || nh % nkv != 0 || pages_per_split < 0 || n_splits <= 0) return IL_BAD_ARG;
    const long long rows = (long long)n_decode * nh * n_splits;
    if (rows > IL_NOALLOC_MAX_ROWS) return IL_NOALLOC_TOO_LARGE;
    if (n_splits > AD_MAX_SPLITS) return IL_NOALLOC_TOO_LARGE;

    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= IL_NOALLOC_MAX_DEVICES) return IL_NOALLOC_NO_SYMBOL;
    if (!il_noalloc_addr[dev]) {
        // In host code the array's name stands for the symbol, not for a device address: ask the
        // runtime for the address on the current device, once, and keep it.
        float* p = nullptr;
        if (cudaGetSymbolAddress((void**)&p, il_noalloc_scratch) != cudaSuccess || !p) return IL_NOALLOC_NO_SYMBOL;
        il_noalloc_addr[dev] = p;
    }
    float* o_part = il_noalloc_addr[dev];
    float* ml_part = o_part + (size_t)IL_NOALLOC_MAX_ROWS * HEAD_DIM;
    return ad_launch(qkv, row_stride, out, cache, block_table, bt_stride, entry_kvlen, n_decode, nh, nkv, scale, window,
                     pages_per_split, n_splits, o_part, ml_part, stream);
}

extern "C" __attribute__((visibility("default")))
const char* il_attn_decode_noalloc_strerror(int code) {
    switch (code) {
        case IL_OK: return "launched";
        case IL_BAD_ARG: return "bad argument (head counts, splits)";
        case IL_UNSUPPORTED: return "head_dim or page size differs from what this library was compiled for";
        case IL_NOALLOC_TOO_LARGE:
            return "n_decode * n_heads * n_splits exceeds IL_NOALLOC_MAX_ROWS: the built-in scratch array is too small "
                   "for this call; use fewer splits or a smaller batch, or il_attn_decode with your own scratch";
        case IL_NOALLOC_NO_SYMBOL: return "the device address of the built-in scratch array could not be obtained";
        default: return code >= 1000 ? "a CUDA call failed (code - 1000 is the cudaError_t)" : "unknown code";
    }
}

extern "C" __attribute__((visibility("default"))) int il_attn_decode_noalloc_max_rows(void) { return IL_NOALLOC_MAX_ROWS; }
extern "C" __attribute__((visibility("default"))) long long il_attn_decode_noalloc_scratch_bytes(void) {
    return (long long)sizeof(float) * IL_NOALLOC_MAX_ROWS * (HEAD_DIM + 2);
}
