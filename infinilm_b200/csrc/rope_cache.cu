// Rotary position encoding of q and k in place (rotate-half pairing (i, i + rot/2)), then the
// write of the rotated k and of v into the paged cache. Angles are pos * inv_freq[i] in f32;
// cos and sin are multiplied by `mscale` (1 unless a LongRoPE configuration extends the context).
//
// qkv row layout: [nh heads of q | nkv heads of k | nkv heads of v], each head_dim wide.
// Cache layout of one layer: [page][0=K,1=V][kv head][slot in page][head_dim].
// A token's slot follows from its entry's block-table row and its absolute position.
#include "common.cuh"

template <typename TA>
__global__ void rope_store_kernel(TA* __restrict__ qkv, int row_stride, const int* __restrict__ tok_pos,
                                  const int* __restrict__ tok_entry, const int* __restrict__ block_table,
                                  int bt_stride, TA* __restrict__ cache, int page_size, int nh, int nkv, int hd,
                                  int rot, const float* __restrict__ inv_freq, float mscale) {
    const int t = blockIdx.x;
    const int pos = tok_pos[t];
    TA* row = qkv + (size_t)t * row_stride;
    const int half = rot >> 1;
    if (half > 0) {
        const int n_pairs = (nh + nkv) * half;
        for (int idx = threadIdx.x; idx < n_pairs; idx += blockDim.x) {
            const int j = idx / half, i = idx - j * half;
            TA* base = row + (size_t)j * hd;
            const float ang = (float)pos * inv_freq[i];
            float s, c;
            sincosf(ang, &s, &c);
            s *= mscale;
            c *= mscale;
            const float x1 = il_to_f(base[i]), x2 = il_to_f(base[i + half]);
            base[i] = il_from_f<TA>(x1 * c - x2 * s);
            base[i + half] = il_from_f<TA>(x2 * c + x1 * s);
        }
    }
    if (!cache) return;
    __syncthreads();
    const int e = tok_entry[t];
    const int page = block_table[(size_t)e * bt_stride + pos / page_size];
    if (page < 0) return;  // the host reserves every page a step touches; never write elsewhere
    const int off = pos % page_size;
    const TA* ksrc = row + (size_t)nh * hd;
    const TA* vsrc = ksrc + (size_t)nkv * hd;
    const size_t page_elems = (size_t)2 * nkv * page_size * hd;
    TA* kdst = cache + (size_t)page * page_elems;
    TA* vdst = kdst + (size_t)nkv * page_size * hd;
    for (int idx = threadIdx.x; idx < nkv * hd; idx += blockDim.x) {
        const int g = idx / hd, d = idx - g * hd;
        const size_t o = ((size_t)g * page_size + off) * hd + d;
        kdst[o] = ksrc[idx];
        vdst[o] = vsrc[idx];
    }
}

IL_EXPORT int il_rope_store(void* qkv, int act_kind, int row_stride, const int* tok_pos, const int* tok_entry,
                            const int* block_table, int bt_stride, void* cache, int page_size, int T, int nh,
                            int nkv, int hd, int rot, const float* inv_freq, float mscale, cudaStream_t stream) {
    if (T <= 0) return IL_OK;
    if (nh <= 0 || nkv <= 0 || hd <= 0 || rot < 0 || rot > hd || (rot & 1) || page_size <= 0) return IL_BAD_ARG;
    if (row_stride < (nh + 2 * nkv) * hd) return IL_BAD_ARG;
    const int threads = 256;
    if (act_kind == IL_F32)
        rope_store_kernel<float><<<T, threads, 0, stream>>>((float*)qkv, row_stride, tok_pos, tok_entry, block_table, bt_stride,
                                                            (float*)cache, page_size, nh, nkv, hd, rot, inv_freq, mscale);
    else if (act_kind == IL_BF16)
        rope_store_kernel<__nv_bfloat16><<<T, threads, 0, stream>>>((__nv_bfloat16*)qkv, row_stride, tok_pos, tok_entry, block_table,
                                                                    bt_stride, (__nv_bfloat16*)cache, page_size, nh, nkv, hd, rot,
                                                                    inv_freq, mscale);
    else
        return IL_BAD_ARG;
    IL_LAUNCH_CHECK();
    return IL_OK;
}
