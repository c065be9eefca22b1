// Rotary position encoding of q and k in place (rotate-half pairing (i, i + rot/2)), then the
// write of the rotated k and of v into the paged cache. Angles are pos * inv_freq[i] in f32;
// cos and sin are multiplied by `mscale` (1 unless a LongRoPE configuration extends the context).
//
// qkv row layout: [nh heads of q | nkv heads of k | nkv heads of v], each head_dim wide.
// Cache layout of one layer: [page][0=K,1=V][kv head][slot in page][head_dim].
// A token's slot follows from its entry's block-table row and its absolute position.
#include "common.cuh"

__device__ __forceinline__ float2 ld2(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ float2 ld2(const __nv_bfloat16* p) { return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p)); }
__device__ __forceinline__ void st2(float* p, float2 v) { *reinterpret_cast<float2*>(p) = v; }
__device__ __forceinline__ void st2(__nv_bfloat16* p, float2 v) { *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v.x, v.y); }

template <typename TA>
__global__ void rope_store_kernel(TA* __restrict__ qkv, int row_stride, const int* __restrict__ tok_pos,
                                  const int* __restrict__ tok_entry, const int* __restrict__ block_table,
                                  int bt_stride, TA* __restrict__ cache, int page_size, int nh, int nkv, int hd,
                                  int rot, const float* __restrict__ inv_freq, float mscale) {
    il_pdl_begin();
    const int t = blockIdx.x;
    const int pos = tok_pos[t];
    TA* row = qkv + (size_t)t * row_stride;
    const int half = rot >> 1;
    __shared__ float cs[128], sn[128];            // rot <= head_dim <= 256
    if (half > 0) {
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            float s, c;
            sincosf((float)pos * inv_freq[i], &s, &c);
            sn[i] = s * mscale;
            cs[i] = c * mscale;
        }
        __syncthreads();
        if ((half & 1) == 0) {                    // two neighbouring pairs per thread, 4- or 8-byte accesses
            const int hp = half >> 1, n2 = (nh + nkv) * hp;
            for (int idx = threadIdx.x; idx < n2; idx += blockDim.x) {
                const int j = idx / hp, i = (idx - j * hp) * 2;
                TA* base = row + (size_t)j * hd;
                const float2 a = ld2(base + i), b = ld2(base + i + half);
                const float s0 = sn[i], c0 = cs[i], s1 = sn[i + 1], c1 = cs[i + 1];
                st2(base + i, make_float2(a.x * c0 - b.x * s0, a.y * c1 - b.y * s1));
                st2(base + i + half, make_float2(b.x * c0 + a.x * s0, b.y * c1 + a.y * s1));
            }
        } else {
            const int n_pairs = (nh + nkv) * half;
            for (int idx = threadIdx.x; idx < n_pairs; idx += blockDim.x) {
                const int j = idx / half, i = idx - j * half;
                TA* base = row + (size_t)j * hd;
                const float s = sn[i], c = cs[i];
                const float x1 = il_to_f(base[i]), x2 = il_to_f(base[i + half]);
                base[i] = il_from_f<TA>(x1 * c - x2 * s);
                base[i + half] = il_from_f<TA>(x2 * c + x1 * s);
            }
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
    constexpr int VEC = 16 / sizeof(TA);          // elements per 16-byte chunk; head_dim is a multiple of 16
    const int cpr = hd / VEC;
    for (int idx = threadIdx.x; idx < nkv * cpr; idx += blockDim.x) {
        const int g = idx / cpr, c = idx - g * cpr;
        const size_t o = ((size_t)g * page_size + off) * hd + (size_t)c * VEC;
        *reinterpret_cast<uint4*>(kdst + o) = *reinterpret_cast<const uint4*>(ksrc + (size_t)g * hd + (size_t)c * VEC);
        *reinterpret_cast<uint4*>(vdst + o) = *reinterpret_cast<const uint4*>(vsrc + (size_t)g * hd + (size_t)c * VEC);
    }
}

IL_EXPORT int il_rope_store(void* qkv, int act_kind, int row_stride, const int* tok_pos, const int* tok_entry,
                            const int* block_table, int bt_stride, void* cache, int page_size, int T, int nh,
                            int nkv, int hd, int rot, const float* inv_freq, float mscale, cudaStream_t stream) {
    if (T <= 0) return IL_OK;
    if (hd > 256) return IL_UNSUPPORTED;
    if (nh <= 0 || nkv <= 0 || hd <= 0 || rot < 0 || rot > hd || (rot & 1) || page_size <= 0) return IL_BAD_ARG;
    if (row_stride < (nh + 2 * nkv) * hd || hd % 16 != 0 || row_stride % 8 != 0) return IL_BAD_ARG;
    const int threads = 256;
    if (act_kind == IL_F32)
        IL_LAUNCH(rope_store_kernel<float>, T, threads, 0, stream, (float*)qkv, row_stride, tok_pos, tok_entry, block_table, bt_stride,
                                                            (float*)cache, page_size, nh, nkv, hd, rot, inv_freq, mscale);
    else if (act_kind == IL_BF16)
        IL_LAUNCH(rope_store_kernel<__nv_bfloat16>, T, threads, 0, stream, (__nv_bfloat16*)qkv, row_stride, tok_pos, tok_entry, block_table,
                                                                    bt_stride, (__nv_bfloat16*)cache, page_size, nh, nkv, hd, rot,
                                                                    inv_freq, mscale);
    else
        return IL_BAD_ARG;
    IL_LAUNCH_CHECK();
    return IL_OK;
}
