// Token embedding: gathers table rows, multiplies by the embedding scale in f32 and writes the
// f32 residual stream. With round_bf16 the product is rounded to bfloat16 first, which is the
// value a table pre-scaled in bfloat16 would hold.
#include "common.cuh"

template <typename TW>
__global__ void embed_kernel(const int* __restrict__ ids, const TW* __restrict__ table, float scale,
                             float* __restrict__ out, int H, int V, int round_bf16) {
    il_pdl_begin();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (size_t)t * H;
    if (id < 0 || id >= V) {  // the host rejects such ids before launch; never read out of range
        for (int h = threadIdx.x; h < H; h += blockDim.x) o[h] = __int_as_float(0x7fc00000);
        return;
    }
    const TW* row = table + (size_t)id * H;
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        float v = il_to_f(row[h]) * scale;
        if (round_bf16) v = __bfloat162float(__float2bfloat16_rn(v));
        o[h] = v;
    }
}

IL_EXPORT int il_embed(const int* ids, const void* table, int table_kind, float scale, float* out,
                       int T, int H, int V, int round_bf16, cudaStream_t stream) {
    if (T <= 0) return IL_OK;
    if (H <= 0 || V <= 0) return IL_BAD_ARG;
    const int threads = H >= 1024 ? 256 : 128;
    if (table_kind == IL_F32)
        IL_LAUNCH(embed_kernel<float>, T, threads, 0, stream, ids, (const float*)table, scale, out, H, V, round_bf16);
    else if (table_kind == IL_BF16)
        IL_LAUNCH(embed_kernel<__nv_bfloat16>, T, threads, 0, stream, ids, (const __nv_bfloat16*)table, scale, out, H, V, round_bf16);
    else
        return IL_BAD_ARG;
    IL_LAUNCH_CHECK();
    return IL_OK;
}

// token_ids[rows[i]] = src[src_idx[i]]: puts tokens that were sampled on the device (and not read by the host yet)
// into the next step's token list. Out-of-vocabulary values are caught by the gather above.
__global__ void patch_tokens_kernel(int* __restrict__ token_ids, const int* __restrict__ rows, const int* __restrict__ src_idx,
                                    const int* __restrict__ src, int n) {
    il_pdl_begin();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) token_ids[rows[i]] = src[src_idx[i]];
}

IL_EXPORT int il_patch_tokens(int* token_ids, const int* rows, const int* src_idx, const int* src, int n, cudaStream_t stream) {
    if (n <= 0) return IL_OK;
    IL_LAUNCH(patch_tokens_kernel, (n + 127) / 128, 128, 0, stream, token_ids, rows, src_idx, src, n);
    IL_LAUNCH_CHECK();
    return IL_OK;
}
