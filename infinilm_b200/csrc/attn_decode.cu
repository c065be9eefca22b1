// Decode attention over the paged cache in bfloat16: one query token per request, the query heads
// of a kv head packed as the 16 rows of a tensor-core tile, the keys of a request split over
// blocks (split-KV) and merged by a second kernel.
//
//   grid  (splits, kv heads * row tiles, entries), 4 warps per block.
//   A warp walks pages p0+w, p0+w+4, ... of its split with its own pipeline of asynchronous
//   copies (STAGES pages in flight), computes S = Q.K^T (f32), an online softmax in f32 (base 2,
//   scale folded in), and O += P.V with P rounded to bfloat16. The four warps merge in shared
//   memory and the block writes one partial (O unnormalised, running max, sum) per split.
//   A second, wide kernel merges the splits' partials and writes the bfloat16 output.
//
// Token t (= entry t; decode entries come first in a step) has kv length entry_kvlen[t]; its query
// sits at position kvlen-1 and sees positions max(0, kvlen-window) .. kvlen-1 (window <= 0: all).
//
// Two ways of bringing pages into shared memory. With a tensor map of the layer's cache (head_dim a
// multiple of 64) one lane per warp issues TMA tensor copies with the 128-byte swizzle, [16 keys x 64]
// boxes completing on the warp's own mbarriers, and ldmatrix reads the swizzled tiles; small per-lane
// cp.async copies top out near 3 TB/s on this part, the tensor copies do not. Without a map (other
// head sizes) the per-lane cp.async path with padded rows is used.
#include <cuda.h>
#include <cstring>

#include "attn_mma.cuh"

constexpr int AD_WARPS = 4;
constexpr int AD_PAGE = 16;                       // keys per tile = page size this kernel takes
constexpr int AD_STAGES = 2;                      // 4 warps x 2 stages of a page (8-9 KB at head_dim 128): three blocks fit on an SM
constexpr int AD_STAGE_BYTES = 2 * AD_PAGE * AT_ROW_BYTES;
constexpr int AD_SMEM_PIPE = AD_WARPS * AD_STAGES * AD_STAGE_BYTES;
constexpr int AD_SMEM_MERGE = AD_WARPS * 16 * (HEAD_DIM + 4 + 2) * 4;   // the warps' scaled outputs and (m, l)
constexpr int AD_SMEM = (AD_SMEM_PIPE > AD_SMEM_MERGE ? AD_SMEM_PIPE : AD_SMEM_MERGE) + AD_WARPS * AD_STAGES * 8 + 1024;
constexpr bool AD_TMA_OK = (HEAD_DIM % 64 == 0);
constexpr int AD_BOXES = HEAD_DIM / 64;           // 64-column boxes of a K (or V) block
constexpr int AD_TMA_STAGE_BYTES = 2 * AD_BOXES * 2048;   // K boxes then V boxes, each [16 x 64] bf16 = 2 KB
constexpr unsigned AD_SPIN_LIMIT = 1u << 26;

__device__ __forceinline__ bool ad_mbar_wait(uint32_t bar, uint32_t parity) {
    for (unsigned spin = 0; spin < AD_SPIN_LIMIT; ++spin) {
        uint32_t done;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
// One page of one kv head, K and V, all of head_dim: a box of a five-dimensional view of the cache (see il_attn_decode_kv_map).
__device__ __forceinline__ void ad_tma_page(uint32_t dst, const CUtensorMap* map, int g, int page, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %3, %3, %4, %5}], [%2];\n"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(0), "r"(g), "r"(page * 2) : "memory");
}
__device__ __forceinline__ void ad_tma_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
// Address of the 16-byte chunk `ch` of row `r` in a block of [16 x head_dim] stored as 64-column boxes with the 128-byte swizzle.
__device__ __forceinline__ uint32_t ad_swz(uint32_t block, int r, int ch) {
    return block + (ch >> 3) * 2048 + r * 128 + (((ch & 7) ^ (r & 7)) << 4);
}

constexpr int AD_MAX_SPLITS = 128;

// WPR warps merge the splits of one (token, head) row; warp `sub` of them takes splits sub, sub + WPR, ... Every load is
// issued before anything waits for one: the partial outputs of the warp's first sixteen splits (each lane four columns),
// then the (maximum, sum) pairs of all splits in one pass (lanes over splits), and only then the arithmetic. The split
// factors exp2(m_s - M) go through `fs` (shared memory, AD_MAX_SPLITS floats of this warp). With WPR = 4 a row's
// warps leave their sums in `comb` and warp 0 adds them in warp order: with many splits (few requests) the merge is a
// chain of memory round trips, one per sixteen splits of a warp, and four warps make it one.
constexpr int AD_MERGE_ROUND = 16;
#ifndef AD_MERGE_WIDE_FROM
#define AD_MERGE_WIDE_FROM 8                      // more splits than this: four warps a row
#endif

template <int WPR>
__device__ __forceinline__ void ad_merge_row(float* fs, float* comb, const float* o_part, const float* ml_part, size_t row, int n_valid,
                                             int n_splits, __nv_bfloat16* __restrict__ out, int lane, int sub) {
    const size_t pr0 = row * n_splits;
    const int d_first = lane * 4;
    float4 v[AD_MERGE_ROUND];
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < AD_MERGE_ROUND; ++i) {
        const int s_ = sub + WPR * i;
        v[i] = (d_first < AT_HD && s_ < n_valid) ? *reinterpret_cast<const float4*>(o_part + (pr0 + s_) * AT_HD + d_first) : zero4;
    }
    constexpr int PER_LANE = AD_MAX_SPLITS / 32;
    float2 ml[PER_LANE];
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
        const int s_ = lane + 32 * i;
        ml[i] = s_ < n_valid ? *reinterpret_cast<const float2*>(ml_part + (pr0 + s_) * 2) : make_float2(-INFINITY, 0.f);
    }
    float M = -INFINITY;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) M = fmaxf(M, ml[i].x);
    M = il_warp_max(M);
    float L = 0.f;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
        const int s_ = lane + 32 * i;
        const float f = (ml[i].x == -INFINITY) ? 0.f : exp2f(ml[i].x - M);
        if (s_ < n_valid) fs[s_] = f;
        L += f * ml[i].y;
    }
    L = il_warp_sum(L);
    __syncwarp();
    const float inv = 1.f / L;
    for (int d = d_first; d < AT_HD; d += 128) {
        float4 acc = zero4;
        for (int i0 = 0; sub + WPR * i0 < n_valid; i0 += AD_MERGE_ROUND) {
            if (d != d_first || i0 != 0) {        // (the first round is on its way since the start)
#pragma unroll
                for (int i = 0; i < AD_MERGE_ROUND; ++i) {
                    const int s_ = sub + WPR * (i0 + i);
                    v[i] = s_ < n_valid ? *reinterpret_cast<const float4*>(o_part + (pr0 + s_) * AT_HD + d) : zero4;
                }
            }
#pragma unroll
            for (int i = 0; i < AD_MERGE_ROUND; ++i) {    // in the order of the warp's splits: the same sum whatever the round
                const int s_ = sub + WPR * (i0 + i);
                const float f = s_ < n_valid ? fs[s_] : 0.f;
                acc.x += f * v[i].x;
                acc.y += f * v[i].y;
                acc.z += f * v[i].z;
                acc.w += f * v[i].w;
            }
        }
        if (WPR == 1) {
            const uint32_t a = at_pack_bf16(acc.x * inv, acc.y * inv), b = at_pack_bf16(acc.z * inv, acc.w * inv);
            *reinterpret_cast<uint2*>(out + row * AT_HD + d) = make_uint2(a, b);
        } else {
            *reinterpret_cast<float4*>(comb + sub * AT_HD + d) = acc;
        }
    }
    if (WPR > 1) {
        __syncthreads();                          // a block is one row: all its warps are here
        if (sub == 0) {
            for (int d = d_first; d < AT_HD; d += 128) {
                float4 acc = *reinterpret_cast<const float4*>(comb + d);
#pragma unroll
                for (int w = 1; w < WPR; ++w) {
                    const float4 t = *reinterpret_cast<const float4*>(comb + w * AT_HD + d);
                    acc.x += t.x, acc.y += t.y, acc.z += t.z, acc.w += t.w;
                }
                const uint32_t a = at_pack_bf16(acc.x * inv, acc.y * inv), b = at_pack_bf16(acc.z * inv, acc.w * inv);
                *reinterpret_cast<uint2*>(out + row * AT_HD + d) = make_uint2(a, b);
            }
        }
    }
    __syncwarp();
}

// (qkv, and o_part / ml_part in the merge, are written by the kernel before and read after a wait that is not the
// kernel's first statement: they are not declared __restrict__, so that no load of them is treated as read-only
// data and scheduled above the wait.)
__global__ void __launch_bounds__(AD_WARPS * 32) attn_decode_kernel(
    const __nv_bfloat16* qkv, int row_stride, const __nv_bfloat16* __restrict__ cache,
    const int* __restrict__ block_table, int bt_stride, const int* __restrict__ entry_kvlen, int nh, int nkv,
    float scale_log2, int window, int pages_per_split, int n_splits, float* __restrict__ o_part,
    float* __restrict__ ml_part, const __grid_constant__ CUtensorMap kv_map, const __grid_constant__ CUtensorMap kv_page_map,
    int use_tma, int* __restrict__ status, __nv_bfloat16* __restrict__ out_direct) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    // Lengths, block tables and the pages of earlier tokens do not come from the kernel before this one (it writes q and
    // the newest token's slot in the last page): what depends only on them is done before waiting for that kernel.
    const int split = blockIdx.x;
    const int G = nh / nkv;
    const int row_tiles = (G + 15) / 16;
    const int g = blockIdx.y / row_tiles, rt = blockIdx.y - g * row_tiles;
    const int e = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    const int kvlen = entry_kvlen[e];
    if (kvlen <= 0) {                             // no keys: the merge kernel writes zeros for this row, or, where there is none, this block
        if (out_direct) {
            const int h0 = g * G + rt * 16, rv = min(16, G - rt * 16);
            for (int idx = threadIdx.x; idx < rv * (AT_HD / 4); idx += AD_WARPS * 32) {
                const int r = idx / (AT_HD / 4), d = (idx - r * (AT_HD / 4)) * 4;
                *reinterpret_cast<uint2*>(out_direct + ((size_t)e * nh + h0 + r) * AT_HD + d) = make_uint2(0u, 0u);
            }
        }
        return;
    }
    const int lo = (window > 0 && kvlen - window > 0) ? kvlen - window : 0;
    const int first_page = lo / AD_PAGE, last_page = (kvlen - 1) / AD_PAGE;
    // pages_per_split 0: this request's pages are divided evenly over the splits
    if (pages_per_split <= 0) pages_per_split = (last_page - first_page + n_splits) / n_splits;
    const int p0 = first_page + split * pages_per_split;
    int p1 = p0 + pages_per_split;
    if (p1 > last_page + 1) p1 = last_page + 1;
    if (p0 > last_page) return;                   // this split has no keys: the merge kernel knows

    const int* bt = block_table + (size_t)e * bt_stride;
    const size_t page_elems = (size_t)2 * nkv * AD_PAGE * AT_HD;
    const int head0 = g * G + rt * 16;            // first query head of this row tile
    const int rows_valid = min(16, G - rt * 16);

    float o[AT_NT][4];
#pragma unroll
    for (int i = 0; i < AT_NT; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[i][j] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    const int n_my = (p1 - p0 - warp + AD_WARPS - 1) / AD_WARPS;   // pages p0+warp, +4, ...
    // Page ids of this warp's iterations, 32 at a time: lane l holds the id of iteration base + l, so the
    // table lookup is off the path that issues the copies.
    int ids_base = 0;
    int my_ids = (lane < n_my) ? bt[p0 + warp + lane * AD_WARPS] : 0;
    auto page_of = [&](int it) {
        if (it >= ids_base + 32) {
            ids_base += 32;
            my_ids = (ids_base + lane < n_my) ? bt[p0 + warp + (ids_base + lane) * AD_WARPS] : 0;
        }
        return __shfl_sync(0xffffffffu, my_ids, it - ids_base);
    };
    // A block table may hold -1 (a page given back, or a caller's mistake): such a page is never dereferenced. Its
    // copy reads page 0 instead and its keys are masked; bit (it % 32) remembers that from issue to use.
    unsigned bad_pages = 0;
    auto checked_page = [&](int it) {
        int page = page_of(it);
        if (page < 0) {
            bad_pages |= 1u << (it & 31);
            page = 0;
        } else {
            bad_pages &= ~(1u << (it & 31));
        }
        return page;
    };
    // the tensor-copy pipeline of this warp; its first page is asked for now if it is not the last page of the request
    const bool tma = AD_TMA_OK && use_tma;
    const uint32_t tpipe = (uint32_t)__cvta_generic_to_shared(smem) + warp * AD_STAGES * AD_TMA_STAGE_BYTES;
    const uint32_t tbars = (uint32_t)__cvta_generic_to_shared(smem) + AD_WARPS * AD_STAGES * AD_TMA_STAGE_BYTES + warp * AD_STAGES * 8;
    auto tma_issue = [&](int it) {
        if (it < n_my) {
            const int page = checked_page(it);
            if (lane == 0) {
                const uint32_t st = tpipe + (it % AD_STAGES) * AD_TMA_STAGE_BYTES, bar = tbars + (it % AD_STAGES) * 8;
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // the tile was read by ldmatrix before
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(AD_TMA_STAGE_BYTES) : "memory");
                if (use_tma == 2) {               // the whole page in one copy: copies of 2 KB keep the copy engine below the memory's rate
                    ad_tma_page(st, &kv_page_map, g, page, bar);
                } else {
                    const int rk = ((page * 2) * nkv + g) * AD_PAGE, rv = ((page * 2 + 1) * nkv + g) * AD_PAGE;
#pragma unroll
                    for (int bx = 0; bx < AD_BOXES; ++bx) {
                        ad_tma_2d(st + bx * 2048, &kv_map, bx * 64, rk, bar);
                        ad_tma_2d(st + (AD_BOXES + bx) * 2048, &kv_map, bx * 64, rv, bar);
                    }
                }
            }
        }
    };
    int n_early = 0;                              // iterations whose copies are already under way
    if (tma) {
        if (lane == 0) {
            for (int st = 0; st < AD_STAGES; ++st) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(tbars + st * 8));
            asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        }
        __syncwarp();
        for (; n_early < AD_STAGES && p0 + warp + n_early * AD_WARPS < last_page; ++n_early) tma_issue(n_early);
    }
    il_pdl_begin();

    uint32_t qf[AT_KSTEPS][4];
    const __nv_bfloat16* qbase = qkv + (size_t)e * row_stride;
    at_load_q(qf, [&](int r) { return r < rows_valid ? qbase + (size_t)(head0 + r) * AT_HD : nullptr; }, lane);

    // One page: scores, online softmax, P.V. `qk` fills s[2][4] from the K tile, `pv` adds P.V from the V tile.
    auto softmax_page = [&](float (&s)[2][4], int it, uint32_t (&pf)[4]) {
        const int key0 = (p0 + warp + it * AD_WARPS) * AD_PAGE + (lane & 3) * 2;
        const int hi = ((bad_pages >> (it & 31)) & 1) ? 0 : kvlen;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int key = key0 + nt * 8 + (j & 1);
                s[nt][j] = (key >= lo && key < hi) ? s[nt][j] * scale_log2 : -INFINITY;
            }
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
            if (__any_sync(0xffffffffu, corr != 1.f)) {   // once the running maxima have settled nothing is rescaled
#pragma unroll
                for (int nt = 0; nt < AT_NT; ++nt) {
                    o[nt][2 * h] *= corr;
                    o[nt][2 * h + 1] *= corr;
                }
            }
        }
    };

    if (tma) {
        // ---- tensor copies into swizzled tiles, one mbarrier per warp and stage ----
        const uint32_t pipe = tpipe, bars = tbars;
        auto issue = tma_issue;
        for (int s = n_early; s < AD_STAGES; ++s) issue(s);
        for (int it = 0; it < n_my; ++it) {
            if (!ad_mbar_wait(bars + (it % AD_STAGES) * 8, (it / AD_STAGES) & 1)) {
                if (lane == 0) atomicExch(status, 21);
                break;
            }
            const uint32_t kt = pipe + (it % AD_STAGES) * AD_TMA_STAGE_BYTES, vt = kt + AD_BOXES * 2048;
            float s[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
            {
                const int mat = lane >> 3, rr = lane & 7, key = (mat >> 1) * 8 + rr;
#pragma unroll
                for (int kk = 0; kk < AT_KSTEPS; ++kk) {
                    uint32_t b0, b1, b2, b3;
                    at_ldmatrix_x4(b0, b1, b2, b3, ad_swz(kt, key, kk * 2 + (mat & 1)));
                    at_mma(s[0], qf[kk], b0, b1);
                    at_mma(s[1], qf[kk], b2, b3);
                }
            }
            uint32_t pf[4];
            softmax_page(s, it, pf);
            {
                const int mat = lane >> 3, rr = lane & 7, key = (mat & 1) * 8 + rr;
#pragma unroll
                for (int nt = 0; nt < AT_NT; nt += 2) {
                    uint32_t b0, b1, b2, b3;
                    at_ldmatrix_x4_trans(b0, b1, b2, b3, ad_swz(vt, key, nt + (mat >> 1)));
                    at_mma(o[nt], pf, b0, b1);
                    at_mma(o[nt + 1], pf, b2, b3);
                }
            }
            __syncwarp();
            issue(it + AD_STAGES);                // refill the stage this page came from
        }
    } else {
        // ---- per-lane asynchronous copies into padded tiles ----
        const uint32_t pipe = (uint32_t)__cvta_generic_to_shared(smem) + warp * AD_STAGES * AD_STAGE_BYTES;
        auto issue = [&](int it) {
            if (it < n_my) {
                const int page = checked_page(it);
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
            uint32_t pf[4];
            softmax_page(s, it, pf);
            at_pv_16keys(o, pf, st + AD_PAGE * AT_ROW_BYTES, lane);
            __syncwarp();
        }
        at_cp_wait<0>();
    }
    __syncthreads();                              // the pipeline memory is reused for the merge

    // Merge the four warps. Each puts its rows' (m, l) into shared memory; then every thread knows its rows' common
    // maximum M, scales its part of O by 2^(m - M) in registers and writes it out; then the four parts are added, in
    // warp order, sixteen bytes at a time. (One exponential per row and warp: computing them per output element cost
    // this kernel more than its pages did.)
    float* sm_ml = reinterpret_cast<float*>(smem);                     // [warp][16 rows][m, l]
    float* sm_o = sm_ml + AD_WARPS * 16 * 2;                           // [warp][16 rows][AT_HD + 4]
    constexpr int OS = AT_HD + 4;
    if ((lane & 3) == 0) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = (lane >> 2) + 8 * h;
            sm_ml[(warp * 16 + r) * 2] = m[h];
            sm_ml[(warp * 16 + r) * 2 + 1] = l[h];
        }
    }
    __syncthreads();
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = (lane >> 2) + 8 * h;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < AD_WARPS; ++w) M = fmaxf(M, sm_ml[(w * 16 + r) * 2]);
        const float f = (m[h] == -INFINITY) ? 0.f : exp2f(m[h] - M);
        float* row = sm_o + (size_t)(warp * 16 + r) * OS + (lane & 3) * 2;
#pragma unroll
        for (int nt = 0; nt < AT_NT; ++nt) *reinterpret_cast<float2*>(row + nt * 8) = make_float2(f * o[nt][2 * h], f * o[nt][2 * h + 1]);
    }
    il_pdl_tail();
    __syncthreads();
    for (int idx = threadIdx.x; idx < rows_valid * (AT_HD / 4); idx += AD_WARPS * 32) {
        const int r = idx / (AT_HD / 4), d = (idx - r * (AT_HD / 4)) * 4;
        float4 acc = *reinterpret_cast<const float4*>(sm_o + (size_t)r * OS + d);
#pragma unroll
        for (int w = 1; w < AD_WARPS; ++w) {
            const float4 v = *reinterpret_cast<const float4*>(sm_o + (size_t)(w * 16 + r) * OS + d);
            acc.x += v.x;
            acc.y += v.y;
            acc.z += v.z;
            acc.w += v.w;
        }
        const size_t pr = ((size_t)e * nh + head0 + r) * n_splits + split;
        if (out_direct) {
            // one split: nothing to merge, the row is final. The same arithmetic as the merge of a single part (factor 1,
            // the sum over the warps in warp order, one division), so the bits do not depend on which kernel finished the row.
            float M = -INFINITY, L = 0.f;
#pragma unroll
            for (int w = 0; w < AD_WARPS; ++w) M = fmaxf(M, sm_ml[(w * 16 + r) * 2]);
#pragma unroll
            for (int w = 0; w < AD_WARPS; ++w) {
                const float mw = sm_ml[(w * 16 + r) * 2];
                L += ((mw == -INFINITY) ? 0.f : exp2f(mw - M)) * sm_ml[(w * 16 + r) * 2 + 1];
            }
            const float inv = 1.f / L;
            const uint32_t a = at_pack_bf16(acc.x * inv, acc.y * inv), b = at_pack_bf16(acc.z * inv, acc.w * inv);
            *reinterpret_cast<uint2*>(out_direct + pr * AT_HD + d) = make_uint2(a, b);
            continue;
        }
        *reinterpret_cast<float4*>(o_part + pr * AT_HD + d) = acc;
        if (d == 0) {
            float M = -INFINITY, L = 0.f;
#pragma unroll
            for (int w = 0; w < AD_WARPS; ++w) M = fmaxf(M, sm_ml[(w * 16 + r) * 2]);
#pragma unroll
            for (int w = 0; w < AD_WARPS; ++w) {
                const float mw = sm_ml[(w * 16 + r) * 2];
                L += ((mw == -INFINITY) ? 0.f : exp2f(mw - M)) * sm_ml[(w * 16 + r) * 2 + 1];
            }
            ml_part[pr * 2] = M;
            ml_part[pr * 2 + 1] = L;
        }
    }
}

// The merge: WPR warps per (token, head) row - one where the splits are few, the four of a block where they are many.
template <int WPR>
__global__ void __launch_bounds__(128) attn_decode_merge_kernel(const float* o_part, const float* ml_part,
                                                                const int* __restrict__ entry_kvlen, int nh, int n_rows, int window,
                                                                int pages_per_split, int n_splits, __nv_bfloat16* __restrict__ out) {
    __shared__ float fs[4][AD_MAX_SPLITS];
    __shared__ __align__(16) float comb[WPR > 1 ? WPR * AT_HD : 4];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * (4 / WPR) + warp / WPR;      // = e * nh + head
    // the lengths come with the step's descriptors, not from the kernel before: read them while that one still runs
    const int kvlen = row < n_rows ? entry_kvlen[row / nh] : 1;
    const int lo = (window > 0 && kvlen - window > 0) ? kvlen - window : 0;
    const int n_pages = (kvlen - 1) / AD_PAGE - lo / AD_PAGE + 1;
    if (pages_per_split <= 0) pages_per_split = (n_pages + n_splits - 1) / n_splits;
    int n_valid = (n_pages + pages_per_split - 1) / pages_per_split;
    if (n_valid > n_splits) n_valid = n_splits;
    il_pdl_wait();
    if (row >= n_rows) return;
    if (kvlen <= 0) {                             // no keys: the output is zero
        if (warp % WPR == 0)
            for (int d = lane * 4; d < AT_HD; d += 128) *reinterpret_cast<uint2*>(out + (size_t)row * AT_HD + d) = make_uint2(0u, 0u);
        return;
    }
    ad_merge_row<WPR>(fs[warp], comb, o_part, ml_part, (size_t)row, n_valid, n_splits, out, lane, warp % WPR);
}

// Launches the attention kernel and, for more than one split, the merge. Scratch: o_part float32 [n_decode*nh*n_splits*head_dim], ml_part [n_decode*nh*n_splits*2].
static int ad_launch(const void* qkv, int row_stride, void* out, const void* cache, const int* block_table, int bt_stride,
                     const int* entry_kvlen, int n_decode, int nh, int nkv, float scale, int window, int pages_per_split,
                     int n_splits, float* o_part, float* ml_part, cudaStream_t stream, const CUtensorMap* kv_map = nullptr,
                     int* status = nullptr) {
    static CUtensorMap no_map;                    // passed when there is no map: the kernel does not look at it
    int use_tma = (AD_TMA_OK && kv_map && status) ? 1 : 0;
    if (use_tma) {                                // a second map may follow the first: the page view (all zero: there is none)
        const unsigned char* second = reinterpret_cast<const unsigned char*>(kv_map + 1);
        for (size_t i = 0; i < sizeof(CUtensorMap) && use_tma == 1; ++i)
            if (second[i]) use_tma = 2;
    }
    const CUtensorMap& page_map = use_tma == 2 ? kv_map[1] : no_map;
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
        scale * 1.4426950408889634f, window, pages_per_split, n_splits, o_part, ml_part, use_tma ? *kv_map : no_map, page_map, use_tma, status,
        n_splits == 1 ? (__nv_bfloat16*)out : (__nv_bfloat16*)nullptr);
    if (n_splits == 1) {                          // every row is final as the attention kernel leaves it: no merge
        IL_LAUNCH_CHECK();
        return IL_OK;
    }
    const int n_rows = n_decode * nh;
    if (n_splits > AD_MERGE_WIDE_FROM) {
        IL_LAUNCH(attn_decode_merge_kernel<4>, n_rows, 128, 0, stream, (const float*)o_part, (const float*)ml_part, entry_kvlen, nh, n_rows, window,
                  pages_per_split, n_splits, (__nv_bfloat16*)out);
    } else {
        IL_LAUNCH(attn_decode_merge_kernel<1>, (n_rows + 3) / 4, 128, 0, stream, (const float*)o_part, (const float*)ml_part, entry_kvlen, nh, n_rows,
                  window, pages_per_split, n_splits, (__nv_bfloat16*)out);
    }
    IL_LAUNCH_CHECK();
    return IL_OK;
}

// Blocks of the attention kernel that this device runs at once (blocks per SM from the occupancy calculator x SMs);
// 0 if the query fails. The caller sizes the number of splits by it.
IL_EXPORT int il_attn_decode_resident_blocks() {
    static int cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    if (cached[dev]) return cached[dev];
    int per_sm = 0, sms = 0;
    if (cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AD_SMEM) != cudaSuccess ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attn_decode_kernel, AD_WARPS * 32, AD_SMEM) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    cached[dev] = per_sm * sms;
    return cached[dev];
}

// Scratch the caller provides: o_part float32 [n_decode * nh * n_splits * head_dim], ml_part [n_decode * nh * n_splits * 2].
IL_EXPORT int il_attn_decode(const void* qkv, int row_stride, void* out, const void* cache, const int* block_table,
                             int bt_stride, const int* entry_kvlen, int page_size, int n_decode, int nh, int nkv, int hd,
                             float scale, int window, int pages_per_split, int n_splits, float* o_part, float* ml_part,
                             const void* kv_map, int* status, cudaStream_t stream) {
    if (n_decode <= 0) return IL_OK;
    if (hd != HEAD_DIM || page_size != AD_PAGE) return IL_UNSUPPORTED;
    if (nh <= 0 || nkv <= 0 || nh % nkv != 0 || pages_per_split < 0 || n_splits <= 0) return IL_BAD_ARG;
    if (n_splits > AD_MAX_SPLITS) return IL_UNSUPPORTED;
    return ad_launch(qkv, row_stride, out, cache, block_table, bt_stride, entry_kvlen, n_decode, nh, nkv, scale, window,
                     pages_per_split, n_splits, o_part, ml_part, stream, (const CUtensorMap*)kv_map, status);
}

// Writes two tensor maps (2 x 128 bytes at `out_maps`) of one layer's cache, [pages][2][kv heads][16][head_dim] bfloat16:
// first the cache seen as rows of head_dim, for boxes of [16 rows x 64 columns] with the 128-byte swizzle; then a view
// with the dimensions (64 columns, 16 slots, head_dim / 64 column blocks, kv heads, 2 * pages) whose box is one page
// of one kv head, K and V: it lands in shared memory as the same 2 KB tiles, [K, V][column block][slot][64]. The second
// is all zero if the driver does not take it; so is the third, for the prefill kernel (below). out_maps: 3 x 128 bytes.
// n_rows = pages * 2 * kv heads * 16. Returns 0, or IL_UNSUPPORTED.
IL_EXPORT int il_attn_decode_kv_map(void* out_maps, const void* cache, long long n_rows, int hd, int nkv) {
    if (!AD_TMA_OK || hd != HEAD_DIM || nkv <= 0 || ((uintptr_t)cache & 15)) return IL_UNSUPPORTED;
    typedef CUresult (*encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static encode_fn enc = nullptr;
    if (!enc) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
            return IL_UNSUPPORTED;
        enc = (encode_fn)p;
    }
    CUtensorMap m[3];
    memset(m, 0, sizeof(m));
    {
        cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)n_rows};
        cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
        cuuint32_t box[2] = {64, (cuuint32_t)AD_PAGE};
        cuuint32_t estr[2] = {1, 1};
        CUresult r = enc(&m[0], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(cache), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return 2000 + (int)r;
    }
    {
        const cuuint64_t n_kvpages = (cuuint64_t)(n_rows / ((long long)nkv * AD_PAGE));
        cuuint64_t dims[5] = {64, (cuuint64_t)AD_PAGE, (cuuint64_t)(hd / 64), (cuuint64_t)nkv, n_kvpages};
        cuuint64_t strides[4] = {(cuuint64_t)hd * 2, 128, (cuuint64_t)AD_PAGE * hd * 2, (cuuint64_t)nkv * AD_PAGE * hd * 2};
        cuuint32_t box[5] = {64, (cuuint32_t)AD_PAGE, (cuuint32_t)(hd / 64), 1, 2};
        cuuint32_t estr[5] = {1, 1, 1, 1, 1};
        CUtensorMap t;
        CUresult r = enc(&t, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(cache), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r == CUDA_SUCCESS) m[1] = t;          // else: stays zero, the kernel copies 2 KB boxes
    }
    {
        // 16 slots of one kv head (K or V of a page) as tensor-core tiles: (64 columns, 8 slots, column blocks, 2 groups of
        // 8 slots, 16-slot blocks). The box lands as [group][column block][8 slots][64]: 1 KB tiles of 8 rows, those of one
        // column block head_dim / 64 KB apart - a uniform stride over the pages of a key tile, which a descriptor needs.
        cuuint64_t dims[5] = {64, 8, (cuuint64_t)(hd / 64), 2, (cuuint64_t)(n_rows / AD_PAGE)};
        cuuint64_t strides[4] = {(cuuint64_t)hd * 2, 128, (cuuint64_t)8 * hd * 2, (cuuint64_t)AD_PAGE * hd * 2};
        cuuint32_t box[5] = {64, 8, (cuuint32_t)(hd / 64), 2, 1};
        cuuint32_t estr[5] = {1, 1, 1, 1, 1};
        CUtensorMap t;
        CUresult r = enc(&t, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(cache), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r == CUDA_SUCCESS) m[2] = t;          // else: stays zero; the tensor-memory prefill kernel is then not used
    }
    memcpy(out_maps, m, sizeof(m));
    return IL_OK;
}
