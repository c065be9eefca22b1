// Prefill attention over the paged cache in bfloat16: prompt portions of any length, each token
// attending causally to what its request has in the cache (earlier steps' keys and this step's own).
//
//   A block owns up to 64 rows: TPT consecutive tokens of one entry times the G query heads of one
//   kv head (row r -> token r / G, head r % G), 16 rows per warp. It walks the keys in tiles of
//   64 (four pages of 16), double-buffered with asynchronous copies, computes S = Q.K^T with the
//   tensor cores (f32 accumulation), an online softmax in f32 (base 2, scale folded in) and
//   O += P.V with P rounded to bfloat16. Pages wholly above a warp's last query position, or
//   wholly behind its window, are skipped by that warp.
//
//   grid (tiles, kv heads). Tiles are numbered over the entries [first_entry, n_entries) in
//   order; a block finds its entry by walking entry_qstart.
#include "attn_mma.cuh"

constexpr int AP_WARPS = 4;
constexpr int AP_ROWS = AP_WARPS * 16;
constexpr int AP_PAGE = 16;
constexpr int AP_TILE_PAGES = 4;
constexpr int AP_PAGE_BYTES = 2 * AP_PAGE * AT_ROW_BYTES;        // K tile then V tile of one page
constexpr int AP_STAGE_BYTES = AP_TILE_PAGES * AP_PAGE_BYTES;
constexpr int AP_STAGES = 2;
constexpr int AP_SMEM = AP_STAGES * AP_STAGE_BYTES;

// 2^x on the special-function unit (ex2.approx: -inf gives 0, relative error about 2^-22).
__device__ __forceinline__ float ap_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

__global__ void __launch_bounds__(AP_WARPS * 32) attn_prefill_kernel(
    const __nv_bfloat16* __restrict__ qkv, int row_stride, __nv_bfloat16* __restrict__ out,
    const __nv_bfloat16* __restrict__ cache, const int* __restrict__ block_table, int bt_stride,
    const int* __restrict__ entry_qstart, const int* __restrict__ entry_kvlen, int first_entry, int n_entries, int nh,
    int nkv, float scale_log2, int window, int tpt) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int G = nh / nkv;
    const int g = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // which entry and which tokens
    // Tiles are taken from the last to the first: the last tokens of a prompt have the most keys to
    // visit, and starting the longest blocks first shortens the tail of the launch.
    int tile = (int)gridDim.x - 1 - (int)blockIdx.x, e = first_entry;
    for (; e < n_entries; ++e) {
        const int nt = (entry_qstart[e + 1] - entry_qstart[e] + tpt - 1) / tpt;
        if (tile < nt) break;
        tile -= nt;
    }
    if (e >= n_entries) return;
    const int q0 = entry_qstart[e], q1 = entry_qstart[e + 1];
    const int kvlen = entry_kvlen[e];
    const int start_pos = kvlen - (q1 - q0);      // position of the entry's first token
    const int tok0 = q0 + tile * tpt;             // first token row of this block
    const int n_tok = min(tpt, q1 - tok0);
    const int rows_valid = n_tok * G;
    const int* bt = block_table + (size_t)e * bt_stride;
    const size_t page_elems = (size_t)2 * nkv * AP_PAGE * AT_HD;

    // this thread's two rows: r0 = 16*warp + lane/4, r1 = r0 + 8
    int rpos[2], rlo[2];
    bool rvalid[2];
    const __nv_bfloat16* qptr[2];
    __nv_bfloat16* optr[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = warp * 16 + (lane >> 2) + 8 * h;
        rvalid[h] = r < rows_valid;
        const int tl = rvalid[h] ? r / G : 0, hh = rvalid[h] ? r - tl * G : 0;
        rpos[h] = start_pos + (tok0 - q0) + tl;
        rlo[h] = (window > 0 && rpos[h] - window + 1 > 0) ? rpos[h] - window + 1 : 0;
        qptr[h] = rvalid[h] ? qkv + (size_t)(tok0 + tl) * row_stride + (size_t)(g * G + hh) * AT_HD : nullptr;
        optr[h] = rvalid[h] ? out + (size_t)(tok0 + tl) * nh * AT_HD + (size_t)(g * G + hh) * AT_HD : nullptr;
        if (!rvalid[h]) { rpos[h] = -1; rlo[h] = 0; }
    }
    uint32_t qf[AT_KSTEPS][4];
    {
        const __nv_bfloat16* r0 = qptr[0];
        const __nv_bfloat16* r1 = qptr[1];
        const int c = (lane & 3) * 2;
#pragma unroll
        for (int kk = 0; kk < AT_KSTEPS; ++kk) {
            qf[kk][0] = r0 ? *reinterpret_cast<const uint32_t*>(r0 + kk * 16 + c) : 0u;
            qf[kk][1] = r1 ? *reinterpret_cast<const uint32_t*>(r1 + kk * 16 + c) : 0u;
            qf[kk][2] = r0 ? *reinterpret_cast<const uint32_t*>(r0 + kk * 16 + c + 8) : 0u;
            qf[kk][3] = r1 ? *reinterpret_cast<const uint32_t*>(r1 + kk * 16 + c + 8) : 0u;
        }
    }
    // warp-wide and block-wide key ranges
    int wmax = max(rpos[0], rpos[1]);
    int wmin_lo = min(rvalid[0] ? rlo[0] : 0x7fffffff, rvalid[1] ? rlo[1] : 0x7fffffff);
    int wmin_pos = min(rpos[0], rpos[1]);         // -1 when a row of the warp is not valid: such a warp always masks
    int wmax_lo = max(rlo[0], rlo[1]);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        wmax = max(wmax, __shfl_xor_sync(0xffffffffu, wmax, off));
        wmin_lo = min(wmin_lo, __shfl_xor_sync(0xffffffffu, wmin_lo, off));
        wmin_pos = min(wmin_pos, __shfl_xor_sync(0xffffffffu, wmin_pos, off));
        wmax_lo = max(wmax_lo, __shfl_xor_sync(0xffffffffu, wmax_lo, off));
    }
    const int bpos_first = start_pos + (tok0 - q0), bpos_last = bpos_first + n_tok - 1;
    const int blo = (window > 0 && bpos_first - window + 1 > 0) ? bpos_first - window + 1 : 0;
    const int page_first = blo / AP_PAGE, page_last = bpos_last / AP_PAGE;
    const int n_tiles = (page_last - page_first) / AP_TILE_PAGES + 1;

    float o[AT_NT][4];
#pragma unroll
    for (int i = 0; i < AT_NT; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[i][j] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(smem);
    auto issue = [&](int it) {                    // warp w copies page w of tile `it`
        if (it < n_tiles) {
            const int pidx = page_first + it * AP_TILE_PAGES + warp;
            if (pidx <= page_last) {
                const int page = bt[pidx];
                const uint32_t st = sbase + (it % AP_STAGES) * AP_STAGE_BYTES + warp * AP_PAGE_BYTES;
                at_load_page(st, st + AP_PAGE * AT_ROW_BYTES, cache + (size_t)page * page_elems, g, nkv, AP_PAGE, 0, AP_PAGE, lane);
            }
        }
        at_cp_commit();
    };
    issue(0);
    for (int it = 0; it < n_tiles; ++it) {
        issue(it + 1);
        at_cp_wait<1>();
        __syncthreads();
        const uint32_t st = sbase + (it % AP_STAGES) * AP_STAGE_BYTES;
        const int key_base = (page_first + it * AP_TILE_PAGES) * AP_PAGE;
        float s[AP_TILE_PAGES][2][4];
        bool use[AP_TILE_PAGES];
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int p = 0; p < AP_TILE_PAGES; ++p) {
            const int k0 = key_base + p * AP_PAGE;
            use[p] = (k0 <= wmax) && (k0 + AP_PAGE - 1 >= wmin_lo);   // the same for the whole warp
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int j = 0; j < 4; ++j) s[p][nt][j] = 0.f;
        }
        // S = Q.K^T for the four pages together: eight independent accumulator chains per k-step
        {
            const int mat = lane >> 3, rr = lane & 7;
            const uint32_t kb = st + ((mat >> 1) * 8 + rr) * AT_ROW_BYTES + (mat & 1) * 16;
#pragma unroll
            for (int kk = 0; kk < AT_KSTEPS; ++kk) {
#pragma unroll
                for (int p = 0; p < AP_TILE_PAGES; ++p) {
                    if (!use[p]) continue;
                    uint32_t b0, b1, b2, b3;
                    at_ldmatrix_x4(b0, b1, b2, b3, kb + p * AP_PAGE_BYTES + kk * 32);
                    at_mma(s[p][0], qf[kk], b0, b1);
                    at_mma(s[p][1], qf[kk], b2, b3);
                }
            }
        }
        // Masks only where a key can lie outside a row's range: above the warp's lowest query position, or below
        // its highest window edge. Scores stay unscaled here; the scale goes into the exponent below.
#pragma unroll
        for (int p = 0; p < AP_TILE_PAGES; ++p) {
            if (!use[p]) continue;
            const int k0 = key_base + p * AP_PAGE;
            const bool need_mask = (k0 + AP_PAGE - 1 > wmin_pos) || (k0 < wmax_lo);
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int h = j >> 1;
                    if (need_mask) {
                        const int key = k0 + nt * 8 + (lane & 3) * 2 + (j & 1);
                        if (!(key <= rpos[h] && key >= rlo[h])) s[p][nt][j] = -INFINITY;
                    }
                    mx[h] = fmaxf(mx[h], s[p][nt][j]);
                }
        }
        float corr[2], msafe[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
            const float mn = fmaxf(m[h], mx[h] * scale_log2);      // running maximum of the scaled scores (scale > 0)
            corr[h] = (mn == -INFINITY) ? 1.f : ap_ex2(m[h] - mn);
            msafe[h] = (mn == -INFINITY) ? 0.f : mn;
            m[h] = mn;
        }
        if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {   // nothing to rescale once the maxima have settled
#pragma unroll
            for (int nt = 0; nt < AT_NT; ++nt) {
                o[nt][0] *= corr[0];
                o[nt][1] *= corr[0];
                o[nt][2] *= corr[1];
                o[nt][3] *= corr[1];
            }
        }
        float rs[2] = {0.f, 0.f};
#pragma unroll
        for (int p = 0; p < AP_TILE_PAGES; ++p) {
            if (!use[p]) continue;
            uint32_t pf[4];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                // 2^(s * scale - m) with one fused multiply-add per score
                const float a = ap_ex2(fmaf(s[p][0][2 * h], scale_log2, -msafe[h])), b = ap_ex2(fmaf(s[p][0][2 * h + 1], scale_log2, -msafe[h]));
                const float c = ap_ex2(fmaf(s[p][1][2 * h], scale_log2, -msafe[h])), d = ap_ex2(fmaf(s[p][1][2 * h + 1], scale_log2, -msafe[h]));
                rs[h] += a + b + c + d;
                pf[h] = at_pack_bf16(a, b);
                pf[2 + h] = at_pack_bf16(c, d);
            }
            at_pv_16keys(o, pf, st + p * AP_PAGE_BYTES + AP_PAGE * AT_ROW_BYTES, lane);
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            rs[h] += __shfl_xor_sync(0xffffffffu, rs[h], 1);
            rs[h] += __shfl_xor_sync(0xffffffffu, rs[h], 2);
            l[h] = l[h] * corr[h] + rs[h];
        }
        __syncthreads();                          // everyone is done with this stage before it is refilled
    }
    at_cp_wait<0>();
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        if (!rvalid[h]) continue;
        const float inv = 1.f / l[h];
        __nv_bfloat16* orow = optr[h];
#pragma unroll
        for (int nt = 0; nt < AT_NT; ++nt) {
            const uint32_t v = at_pack_bf16(o[nt][2 * h] * inv, o[nt][2 * h + 1] * inv);
            *reinterpret_cast<uint32_t*>(orow + nt * 8 + (lane & 3) * 2) = v;
        }
    }
}

// n_tiles_total: sum over entries [first_entry, n_entries) of ceil(q_len / tpt), tpt = max(1, 64 / (nh/nkv)).
IL_EXPORT int il_attn_prefill(const void* qkv, int row_stride, void* out, const void* cache, const int* block_table,
                              int bt_stride, const int* entry_qstart, const int* entry_kvlen, int page_size,
                              int first_entry, int n_entries, int n_tiles_total, int nh, int nkv, int hd, float scale,
                              int window, cudaStream_t stream) {
    if (n_tiles_total <= 0 || first_entry >= n_entries) return IL_OK;
    if (hd != HEAD_DIM || page_size != AP_PAGE) return IL_UNSUPPORTED;
    if (nh <= 0 || nkv <= 0 || nh % nkv != 0) return IL_BAD_ARG;
    const int G = nh / nkv;
    if (G > AP_ROWS) return IL_UNSUPPORTED;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AP_SMEM);
        if (e != cudaSuccess) return 1000 + (int)e;
        attr_set = true;
    }
    dim3 grid(n_tiles_total, nkv);
    attn_prefill_kernel<<<grid, AP_WARPS * 32, AP_SMEM, stream>>>(
        (const __nv_bfloat16*)qkv, row_stride, (__nv_bfloat16*)out, (const __nv_bfloat16*)cache, block_table, bt_stride,
        entry_qstart, entry_kvlen, first_entry, n_entries, nh, nkv, scale * 1.4426950408889634f, window, AP_ROWS / G);
    IL_LAUNCH_CHECK();
    return IL_OK;
}
