// Decode attention over the paged cache in bfloat16: one query token per request, the query heads
// of a kv head packed as the 16 rows of a tensor-core tile, the keys of a request split over
// blocks (split-KV) and merged by a second kernel.
//
//   grid  (splits, kv heads * row tiles, entries), 4 warps per block.
//   A warp walks pages p0+w, p0+w+4, ... of its split with its own pipeline of asynchronous
//   copies (STAGES pages in flight), computes S = Q.K^T (f32), an online softmax in f32 (base 2,
//   scale folded in), and O += P.V with P rounded to bfloat16. The four warps merge in shared
//   memory and the block writes one partial (O unnormalised, running max, sum) per split.
//   il_attn_decode_merge combines the partials of a (token, head) and writes bfloat16 output.
//
// Token t (= entry t; decode entries come first in a step) has kv length entry_kvlen[t]; its query
// sits at position kvlen-1 and sees positions max(0, kvlen-window) .. kvlen-1 (window <= 0: all).
#include "attn_mma.cuh"

constexpr int AD_WARPS = 4;
constexpr int AD_PAGE = 16;                       // keys per tile = page size this kernel takes
constexpr int AD_STAGES = (HEAD_DIM <= 128) ? 3 : 2;      // 4 warps x 3 stages of a page: two blocks fit on an SM at head_dim 128
constexpr int AD_STAGE_BYTES = 2 * AD_PAGE * AT_ROW_BYTES;
constexpr int AD_SMEM_PIPE = AD_WARPS * AD_STAGES * AD_STAGE_BYTES;
constexpr int AD_SMEM_MERGE = AD_WARPS * 16 * (HEAD_DIM + 2) * 4;
constexpr int AD_SMEM = AD_SMEM_PIPE > AD_SMEM_MERGE ? AD_SMEM_PIPE : AD_SMEM_MERGE;

__global__ void __launch_bounds__(AD_WARPS * 32) attn_decode_kernel(
    const __nv_bfloat16* __restrict__ qkv, int row_stride, const __nv_bfloat16* __restrict__ cache,
    const int* __restrict__ block_table, int bt_stride, const int* __restrict__ entry_kvlen, int nh, int nkv,
    float scale_log2, int window, int pages_per_split, int n_splits, float* __restrict__ o_part,
    float* __restrict__ ml_part) {
    extern __shared__ __align__(16) unsigned char smem[];
    il_pdl_launch_dependents();
    il_pdl_wait();
    const int split = blockIdx.x;
    const int G = nh / nkv;
    const int row_tiles = (G + 15) / 16;
    const int g = blockIdx.y / row_tiles, rt = blockIdx.y - g * row_tiles;
    const int e = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    const int kvlen = entry_kvlen[e];
    const int lo = (window > 0 && kvlen - window > 0) ? kvlen - window : 0;
    const int first_page = lo / AD_PAGE, last_page = (kvlen - 1) / AD_PAGE;
    // pages_per_split 0: this request's pages are divided evenly over the splits
    if (pages_per_split <= 0) pages_per_split = (last_page - first_page + n_splits) / n_splits;
    const int p0 = first_page + split * pages_per_split;
    int p1 = p0 + pages_per_split;
    if (p1 > last_page + 1) p1 = last_page + 1;
    if (p0 > last_page) return;                   // this split has no keys; the merge knows

    const int* bt = block_table + (size_t)e * bt_stride;
    const size_t page_elems = (size_t)2 * nkv * AD_PAGE * AT_HD;
    const int head0 = g * G + rt * 16;            // first query head of this row tile
    const int rows_valid = min(16, G - rt * 16);

    uint32_t qf[AT_KSTEPS][4];
    const __nv_bfloat16* qbase = qkv + (size_t)e * row_stride;
    at_load_q(qf, [&](int r) { return r < rows_valid ? qbase + (size_t)(head0 + r) * AT_HD : nullptr; }, lane);

    float o[AT_NT][4];
#pragma unroll
    for (int i = 0; i < AT_NT; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[i][j] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    const uint32_t pipe = (uint32_t)__cvta_generic_to_shared(smem) + warp * AD_STAGES * AD_STAGE_BYTES;
    const int n_my = (p1 - p0 - warp + AD_WARPS - 1) / AD_WARPS;   // pages p0+warp, +4, ...
    // Page ids of this warp's iterations, 32 at a time: lane l holds the id of iteration base + l, so the
    // table lookup is off the path that issues the copies.
    int ids_base = 0;
    int my_ids = (lane < n_my) ? bt[p0 + warp + lane * AD_WARPS] : 0;
    auto issue = [&](int it) {
        if (it < n_my) {
            if (it >= ids_base + 32) {
                ids_base += 32;
                my_ids = (ids_base + lane < n_my) ? bt[p0 + warp + (ids_base + lane) * AD_WARPS] : 0;
            }
            const int page = __shfl_sync(0xffffffffu, my_ids, it - ids_base);
            const uint32_t st = pipe + (it % AD_STAGES) * AD_STAGE_BYTES;
            at_load_page(st, st + AD_PAGE * AT_ROW_BYTES, cache + (size_t)page * page_elems, g, nkv, AD_PAGE, 0, AD_PAGE, lane);
        }
        at_cp_commit();
    };
#pragma unroll
    for (int s = 0; s < AD_STAGES - 1; ++s) issue(s);

    for (int it = 0; it < n_my; ++it) {
        issue(it + AD_STAGES - 1);
        at_cp_wait<AD_STAGES - 1>();
        __syncwarp();
        const uint32_t st = pipe + (it % AD_STAGES) * AD_STAGE_BYTES;
        float s[2][4];
        at_qk_16keys(s, qf, st, lane);
        // mask keys outside [lo, kvlen)
        const int key0 = (p0 + warp + it * AD_WARPS) * AD_PAGE + (lane & 3) * 2;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int key = key0 + nt * 8 + (j & 1);
                s[nt][j] = (key >= lo && key < kvlen) ? s[nt][j] * scale_log2 : -INFINITY;
            }
        uint32_t pf[4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {             // h = 0: row lane/4, h = 1: row lane/4 + 8
            float mx = fmaxf(fmaxf(s[0][2 * h], s[0][2 * h + 1]), fmaxf(s[1][2 * h], s[1][2 * h + 1]));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float mn = fmaxf(m[h], mx);
            const float corr = (mn == -INFINITY) ? 1.f : exp2f(m[h] - mn);
            const float msafe = (mn == -INFINITY) ? 0.f : mn;
            const float p0v = exp2f(s[0][2 * h] - msafe), p1v = exp2f(s[0][2 * h + 1] - msafe);
            const float p2v = exp2f(s[1][2 * h] - msafe), p3v = exp2f(s[1][2 * h + 1] - msafe);
            float rs = p0v + p1v + p2v + p3v;
            rs += __shfl_xor_sync(0xffffffffu, rs, 1);
            rs += __shfl_xor_sync(0xffffffffu, rs, 2);
            l[h] = l[h] * corr + rs;
            m[h] = mn;
            pf[h] = at_pack_bf16(p0v, p1v);       // keys 0-7 of this row
            pf[2 + h] = at_pack_bf16(p2v, p3v);   // keys 8-15
#pragma unroll
            for (int nt = 0; nt < AT_NT; ++nt) {
                o[nt][2 * h] *= corr;
                o[nt][2 * h + 1] *= corr;
            }
        }
        at_pv_16keys(o, pf, st + AD_PAGE * AT_ROW_BYTES, lane);
        __syncwarp();
    }
    at_cp_wait<0>();
    __syncthreads();                              // the pipeline memory is reused for the merge

    // merge the four warps: each writes (m, l, O) for its 16 rows
    float* mo = reinterpret_cast<float*>(smem) + (size_t)warp * 16 * (AT_HD + 2);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = (lane >> 2) + 8 * h;
        float* row = mo + (size_t)r * (AT_HD + 2);
        if ((lane & 3) == 0) {
            row[AT_HD] = m[h];
            row[AT_HD + 1] = l[h];
        }
#pragma unroll
        for (int nt = 0; nt < AT_NT; ++nt) {
            row[nt * 8 + (lane & 3) * 2] = o[nt][2 * h];
            row[nt * 8 + (lane & 3) * 2 + 1] = o[nt][2 * h + 1];
        }
    }
    __syncthreads();
    const float* all = reinterpret_cast<const float*>(smem);
    for (int idx = threadIdx.x; idx < rows_valid * AT_HD; idx += AD_WARPS * 32) {
        const int r = idx / AT_HD, d = idx - r * AT_HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < AD_WARPS; ++w) M = fmaxf(M, all[((size_t)w * 16 + r) * (AT_HD + 2) + AT_HD]);
        float acc = 0.f, L = 0.f;
#pragma unroll
        for (int w = 0; w < AD_WARPS; ++w) {
            const float* row = all + ((size_t)w * 16 + r) * (AT_HD + 2);
            const float f = (row[AT_HD] == -INFINITY) ? 0.f : exp2f(row[AT_HD] - M);
            acc += f * row[d];
            L += f * row[AT_HD + 1];
        }
        const size_t pr = ((size_t)e * nh + head0 + r) * n_splits + split;
        o_part[pr * AT_HD + d] = acc;
        if (d == 0) {
            ml_part[pr * 2] = M;
            ml_part[pr * 2 + 1] = L;
        }
    }
}

constexpr int AD_MAX_SPLITS = 128;

// One warp per (token, head): the split factors exp2(m_s - M) are computed once (lanes over splits)
// and kept in shared memory; then each lane sums four output columns over the splits.
__global__ void __launch_bounds__(128) attn_decode_merge_kernel(const float* __restrict__ o_part, const float* __restrict__ ml_part,
                                                                const int* __restrict__ entry_kvlen, int nh, int n_rows, int window,
                                                                int pages_per_split, int n_splits, __nv_bfloat16* __restrict__ out) {
    __shared__ float fs[4][AD_MAX_SPLITS];
    il_pdl_launch_dependents();
    il_pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * 4 + warp;        // = e * nh + head
    if (row >= n_rows) return;
    const int e = row / nh;
    const int kvlen = entry_kvlen[e];
    const int lo = (window > 0 && kvlen - window > 0) ? kvlen - window : 0;
    const int n_pages = (kvlen - 1) / AD_PAGE - lo / AD_PAGE + 1;
    if (pages_per_split <= 0) pages_per_split = (n_pages + n_splits - 1) / n_splits;
    int n_valid = (n_pages + pages_per_split - 1) / pages_per_split;
    if (n_valid > n_splits) n_valid = n_splits;
    const size_t pr0 = (size_t)row * n_splits;
    float M = -INFINITY;
    for (int s = lane; s < n_valid; s += 32) M = fmaxf(M, ml_part[(pr0 + s) * 2]);
    M = il_warp_max(M);
    float L = 0.f;
    for (int s = lane; s < n_valid; s += 32) {
        const float ms = ml_part[(pr0 + s) * 2];
        const float f = (ms == -INFINITY) ? 0.f : exp2f(ms - M);
        fs[warp][s] = f;
        L += f * ml_part[(pr0 + s) * 2 + 1];
    }
    L = il_warp_sum(L);
    __syncwarp();
    const float inv = 1.f / L;
    for (int d = lane * 4; d < AT_HD; d += 128) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
        for (int s = 0; s < n_valid; ++s) {
            const float4 v = *reinterpret_cast<const float4*>(o_part + (pr0 + s) * AT_HD + d);
            const float f = fs[warp][s];
            acc.x += f * v.x;
            acc.y += f * v.y;
            acc.z += f * v.z;
            acc.w += f * v.w;
        }
        const uint32_t a = at_pack_bf16(acc.x * inv, acc.y * inv), b = at_pack_bf16(acc.z * inv, acc.w * inv);
        *reinterpret_cast<uint2*>(out + (size_t)row * AT_HD + d) = make_uint2(a, b);
    }
}

// Launches both kernels. Scratch: o_part float32 [n_decode*nh*n_splits*head_dim], ml_part [n_decode*nh*n_splits*2].
static int ad_launch(const void* qkv, int row_stride, void* out, const void* cache, const int* block_table, int bt_stride,
                     const int* entry_kvlen, int n_decode, int nh, int nkv, float scale, int window, int pages_per_split,
                     int n_splits, float* o_part, float* ml_part, cudaStream_t stream) {
    static bool attr_set[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AD_SMEM);
        if (e != cudaSuccess) return 1000 + (int)e;
        attr_set[dev] = true;
    }
    const int G = nh / nkv, row_tiles = (G + 15) / 16;
    dim3 grid(n_splits, nkv * row_tiles, n_decode);
    IL_LAUNCH(attn_decode_kernel, grid, AD_WARPS * 32, AD_SMEM, stream,
        (const __nv_bfloat16*)qkv, row_stride, (const __nv_bfloat16*)cache, block_table, bt_stride, entry_kvlen, nh, nkv,
        scale * 1.4426950408889634f, window, pages_per_split, n_splits, o_part, ml_part);
    const int n_rows = n_decode * nh;
    IL_LAUNCH(attn_decode_merge_kernel, (n_rows + 3) / 4, 128, 0, stream, (const float*)o_part, (const float*)ml_part, entry_kvlen, nh, n_rows, window, pages_per_split,
                                                                  n_splits, (__nv_bfloat16*)out);
    IL_LAUNCH_CHECK();
    return IL_OK;
}

// Scratch the caller provides: o_part float32 [n_decode * nh * n_splits * head_dim], ml_part [n_decode * nh * n_splits * 2].
IL_EXPORT int il_attn_decode(const void* qkv, int row_stride, void* out, const void* cache, const int* block_table,
                             int bt_stride, const int* entry_kvlen, int page_size, int n_decode, int nh, int nkv, int hd,
                             float scale, int window, int pages_per_split, int n_splits, float* o_part, float* ml_part,
                             cudaStream_t stream) {
    if (n_decode <= 0) return IL_OK;
    if (hd != HEAD_DIM || page_size != AD_PAGE) return IL_UNSUPPORTED;
    if (nh <= 0 || nkv <= 0 || nh % nkv != 0 || pages_per_split < 0 || n_splits <= 0) return IL_BAD_ARG;
    if (n_splits > AD_MAX_SPLITS) return IL_UNSUPPORTED;
    return ad_launch(qkv, row_stride, out, cache, block_table, bt_stride, entry_kvlen, n_decode, nh, nkv, scale, window,
                     pages_per_split, n_splits, o_part, ml_part, stream);
}
