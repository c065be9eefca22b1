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
    // Positions, block tables and the angle table do not come from the kernel before this one: all of that is done
    // before waiting for it. After the wait a thread reads its pairs once and writes them where they go: q and k back
    // into the row, k and v into the cache slot.
    const int t = blockIdx.x;
    const int pos = tok_pos[t];
    TA* row = qkv + (size_t)t * row_stride;
    const int half = rot >> 1;
    __shared__ float cs[128], sn[128];            // rot <= head_dim <= 256
    TA* kdst = nullptr;                           // this token's K slot of kv head 0, or null: nothing to store
    size_t head_step = 0, v_off = 0;
    if (cache) {
        const int e = tok_entry[t];
        const int page = block_table[(size_t)e * bt_stride + pos / page_size];
        if (page >= 0) {                          // the host reserves every page a step touches; never write elsewhere
            head_step = (size_t)page_size * hd;
            v_off = (size_t)nkv * head_step;
            kdst = cache + (size_t)page * 2 * v_off + (size_t)(pos % page_size) * hd;
        }
    }
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float s, c;
        sincosf((float)pos * inv_freq[i], &s, &c);
        sn[i] = s * mscale;
        cs[i] = c * mscale;
    }
    __syncthreads();
    il_pdl_launch_dependents();                   // the attention kernel behind this one has a prologue of its own to run meanwhile
    il_pdl_wait();
    // After the wait every load of a batch is issued before its first store: the row is read and written in place, so
    // the compiler keeps loads behind earlier stores, and a loop of load-rotate-store rounds would pay the memory
    // latency once per round.
    constexpr int VEC = 16 / sizeof(TA);          // elements per 16-byte chunk; head_dim is a multiple of 16
    const int cpr = hd / VEC;
    const TA* ksrc = row + (size_t)nh * hd;
    const TA* vsrc = ksrc + (size_t)nkv * hd;
    constexpr int UV = 2, UR = 4;
    for (int vb = 0; vb < (kdst ? nkv * cpr : 0) || vb == 0; vb += UV * blockDim.x) {
        uint4 vv[UV];
        const int n_v = kdst ? nkv * cpr : 0;
#pragma unroll
        for (int u = 0; u < UV; ++u) {
            const int idx = vb + u * blockDim.x + threadIdx.x;
            if (idx < n_v) vv[u] = *reinterpret_cast<const uint4*>(vsrc + (size_t)(idx / cpr) * hd + (size_t)(idx % cpr) * VEC);
        }
        if (vb == 0 && half > 0) {
            if ((half & 1) == 0) {                // two neighbouring pairs per thread, 4- or 8-byte accesses
                const int hp = half >> 1, n2 = (nh + nkv) * hp;
                for (int rb = 0; rb < n2; rb += UR * blockDim.x) {
                    float2 a[UR], b[UR];
#pragma unroll
                    for (int u = 0; u < UR; ++u) {
                        const int idx = rb + u * blockDim.x + threadIdx.x;
                        if (idx < n2) {
                            const int j = idx / hp, i = (idx - j * hp) * 2;
                            a[u] = ld2(row + (size_t)j * hd + i);
                            b[u] = ld2(row + (size_t)j * hd + i + half);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < UR; ++u) {
                        const int idx = rb + u * blockDim.x + threadIdx.x;
                        if (idx < n2) {
                            const int j = idx / hp, i = (idx - j * hp) * 2;
                            TA* base = row + (size_t)j * hd;
                            const float s0 = sn[i], c0 = cs[i], s1 = sn[i + 1], c1 = cs[i + 1];
                            const float2 lo = make_float2(a[u].x * c0 - b[u].x * s0, a[u].y * c1 - b[u].y * s1);
                            const float2 hi = make_float2(b[u].x * c0 + a[u].x * s0, b[u].y * c1 + a[u].y * s1);
                            st2(base + i, lo);
                            st2(base + i + half, hi);
                            if (j >= nh && kdst) {
                                TA* kd = kdst + (size_t)(j - nh) * head_step;
                                st2(kd + i, lo);
                                st2(kd + i + half, hi);
                            }
                        }
                    }
                }
            } else {
                const int n_pairs = (nh + nkv) * half;
                for (int idx = threadIdx.x; idx < n_pairs; idx += blockDim.x) {
                    const int j = idx / half, i = idx - j * half;
                    TA* base = row + (size_t)j * hd;
                    const float s = sn[i], c = cs[i];
                    const float x1 = il_to_f(base[i]), x2 = il_to_f(base[i + half]);
                    const TA lo = il_from_f<TA>(x1 * c - x2 * s), hi = il_from_f<TA>(x2 * c + x1 * s);
                    base[i] = lo;
                    base[i + half] = hi;
                    if (j >= nh && kdst) {
                        TA* kd = kdst + (size_t)(j - nh) * head_step;
                        kd[i] = lo;
                        kd[i + half] = hi;
                    }
                }
            }
        }
#pragma unroll
        for (int u = 0; u < UV; ++u) {
            const int idx = vb + u * blockDim.x + threadIdx.x;
            if (idx < n_v)
                *reinterpret_cast<uint4*>(kdst + v_off + (size_t)(idx / cpr) * head_step + (size_t)(idx % cpr) * VEC) = vv[u];
        }
    }
    if (!kdst) return;
    // what the rotation did not touch of k: the dimensions beyond rot (none when rot == head_dim)
    const int tail = hd - rot;
    for (int idx = threadIdx.x; idx < nkv * tail; idx += blockDim.x) {
        const int g = idx / tail, c = rot + (idx - g * tail);
        kdst[(size_t)g * head_step + c] = ksrc[(size_t)g * hd + c];
    }
}

// The same for many tokens (prompt portions): a block's latency does not matter there, how many blocks an SM holds
// does; two passes (rotate in place, then copy k and v to the cache in 16-byte pieces), 256 threads, few registers.
template <typename TA>
__global__ void rope_store_many_kernel(TA* __restrict__ qkv, int row_stride, const int* __restrict__ tok_pos,
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
    constexpr int MANY = 64;                      // from here on: the two-pass kernel for throughput
    if (T > MANY) {
        if (act_kind == IL_F32)
            IL_LAUNCH(rope_store_many_kernel<float>, T, 256, 0, stream, (float*)qkv, row_stride, tok_pos, tok_entry, block_table, bt_stride,
                      (float*)cache, page_size, nh, nkv, hd, rot, inv_freq, mscale);
        else if (act_kind == IL_BF16)
            IL_LAUNCH(rope_store_many_kernel<__nv_bfloat16>, T, 256, 0, stream, (__nv_bfloat16*)qkv, row_stride, tok_pos, tok_entry,
                      block_table, bt_stride, (__nv_bfloat16*)cache, page_size, nh, nkv, hd, rot, inv_freq, mscale);
        else
            return IL_BAD_ARG;
        IL_LAUNCH_CHECK();
        return IL_OK;
    }
    // a thread takes up to four pairs of neighbours at once: enough threads that one round covers a row
    const int pairs2 = (nh + nkv) * (rot / 4);
    int threads = ((pairs2 + 3) / 4 + 31) / 32 * 32;
    threads = threads < 128 ? 128 : (threads > 1024 ? 1024 : threads);
    if (act_kind == IL_F32)
        IL_LAUNCH(rope_store_kernel<float>, T, threads, 0, stream, (float*)qkv, row_stride, tok_pos, tok_entry, block_table, bt_stride,
                  (float*)cache, page_size, nh, nkv, hd, rot, inv_freq, mscale);
    else if (act_kind == IL_BF16)
        IL_LAUNCH(rope_store_kernel<__nv_bfloat16>, T, threads, 0, stream, (__nv_bfloat16*)qkv, row_stride, tok_pos, tok_entry, block_table,
                  bt_stride, (__nv_bfloat16*)cache, page_size, nh, nkv, hd, rot, inv_freq, mscale);
    else
        return IL_BAD_ARG;
    IL_LAUNCH_CHECK();
    return IL_OK;
}
