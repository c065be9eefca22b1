// Plain attention over the paged cache: one warp per (token, query head), keys visited one by
// one with an online softmax in f32. It takes any mix of prompt portions and single decoded
// tokens, any head size up to 256, any number of heads and groups, and an optional window.
// It is the attention of the 32-bit path and the reference beside the fast bfloat16 kernels.
//
// The query of token t is at absolute position p = tok_pos[t] of its request and sees cache
// positions max(0, p - window + 1) .. p (window <= 0: all). Query head j reads kv head j / (nh / nkv).
#include "common.cuh"

#define AP_MAX_PER_LANE 8  // head_dim <= 256

template <typename TA>
__global__ void attn_plain_kernel(const TA* __restrict__ qkv, int row_stride, TA* __restrict__ out,
                                  const TA* __restrict__ cache, const int* __restrict__ block_table, int bt_stride,
                                  const int* __restrict__ tok_pos, const int* __restrict__ tok_entry, int page_size,
                                  int nh, int nkv, int hd, float scale, int window) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int j = blockIdx.y * (blockDim.x >> 5) + warp;
    const int t = blockIdx.x;
    if (j >= nh) return;
    const int g = j / (nh / nkv);
    const int pos = tok_pos[t];
    const int* bt = block_table + (size_t)tok_entry[t] * bt_stride;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;

    float q[AP_MAX_PER_LANE], acc[AP_MAX_PER_LANE];
    const TA* qrow = qkv + (size_t)t * row_stride + (size_t)j * hd;
#pragma unroll
    for (int r = 0; r < AP_MAX_PER_LANE; ++r) {
        const int d = lane + 32 * r;
        q[r] = d < hd ? il_to_f(qrow[d]) : 0.f;
        acc[r] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    const size_t page_elems = (size_t)2 * nkv * page_size * hd;
    for (int kp = lo; kp <= pos; ++kp) {
        const int page = bt[kp / page_size];
        const TA* krow = cache + (size_t)page * page_elems + ((size_t)g * page_size + kp % page_size) * hd;
        const TA* vrow = krow + (size_t)nkv * page_size * hd;
        float dot = 0.f;
#pragma unroll
        for (int r = 0; r < AP_MAX_PER_LANE; ++r) {
            const int d = lane + 32 * r;
            if (d < hd) dot += q[r] * il_to_f(krow[d]);
        }
        dot = il_warp_sum(dot) * scale;
        const float mn = fmaxf(m, dot);
        const float corr = expf(m - mn);  // exp(-inf) = 0 on the first key
        const float p = expf(dot - mn);
        l = l * corr + p;
#pragma unroll
        for (int r = 0; r < AP_MAX_PER_LANE; ++r) {
            const int d = lane + 32 * r;
            if (d < hd) acc[r] = acc[r] * corr + p * il_to_f(vrow[d]);
        }
        m = mn;
    }
    TA* orow = out + (size_t)t * nh * hd + (size_t)j * hd;
    const float inv = 1.f / l;
#pragma unroll
    for (int r = 0; r < AP_MAX_PER_LANE; ++r) {
        const int d = lane + 32 * r;
        if (d < hd) orow[d] = il_from_f<TA>(acc[r] * inv);
    }
}

IL_EXPORT int il_attn_plain(const void* qkv, int act_kind, int row_stride, void* out, const void* cache,
                            const int* block_table, int bt_stride, const int* tok_pos, const int* tok_entry,
                            int page_size, int T, int nh, int nkv, int hd, float scale, int window,
                            cudaStream_t stream) {
    if (T <= 0) return IL_OK;
    if (nh <= 0 || nkv <= 0 || nh % nkv != 0 || hd <= 0 || page_size <= 0) return IL_BAD_ARG;
    if (hd > 32 * AP_MAX_PER_LANE) return IL_UNSUPPORTED;
    const int warps = 4;
    dim3 grid(T, (nh + warps - 1) / warps);
    if (act_kind == IL_F32)
        attn_plain_kernel<float><<<grid, warps * 32, 0, stream>>>((const float*)qkv, row_stride, (float*)out, (const float*)cache,
                                                                  block_table, bt_stride, tok_pos, tok_entry, page_size, nh, nkv,
                                                                  hd, scale, window);
    else if (act_kind == IL_BF16)
        attn_plain_kernel<__nv_bfloat16><<<grid, warps * 32, 0, stream>>>((const __nv_bfloat16*)qkv, row_stride, (__nv_bfloat16*)out,
                                                                          (const __nv_bfloat16*)cache, block_table, bt_stride, tok_pos,
                                                                          tok_entry, page_size, nh, nkv, hd, scale, window);
    else
        return IL_BAD_ARG;
    IL_LAUNCH_CHECK();
    return IL_OK;
}
