// Prefill attention over the paged cache on the 5th-generation tensor cores (head_dim 64 or 128, bfloat16):
// prompt portions of any length, each token attending causally (and inside its window) to what its request
// has in the cache, earlier steps' keys and this step's own.
//
//   A block owns up to 128 rows: TPT consecutive tokens of one entry times the G query heads of one kv head
//   (row r -> token r / G, head r % G), and walks the keys in tiles of 64 (four pages of 16).
//     S = Q.K^T   tcgen05.mma, M 128, N 64, both operands in shared memory (K-major, 128-byte swizzle): Q is put
//                 there once by the softmax threads, K pages arrive as TMA tensor copies. S lives in tensor memory,
//                 two buffers; a buffer is free again as soon as the softmax threads have read it into registers, so
//                 the scores of tile j+2 are computed under the softmax of tile j.
//     softmax     four warps, one thread a row: tcgen05.ld of the row's 64 scores, mask where the tile touches the
//                 row's causal or window edge, base-2 exponent with the scale folded in, f32 sum. The running
//                 maximum is raised only when a tile's maximum is more than 2^8 above it; then the row of O is
//                 rescaled in tensor memory. P goes to shared memory as bfloat16 (a K-major tile like Q's).
//     O += P.V    tcgen05.mma, M 128, N head_dim, A = P from shared memory, B = the V pages as they lie in the
//                 cache (keys by head_dim: MN-major); O accumulates in tensor memory and is divided by the row
//                 sums at the end.
//   Roles by warp: 0 producer (TMA; one copy a page through a view of the cache whose box lands as tensor-core tiles;
//   K and V each in a ring of two slots, K freed as soon as its scores are computed, V when its product is; page ids
//   are read from the block table 32 at a time, ahead of their use), 1 tensor-memory allocation and issue of the
//   score products, 2 issue of the output products, 3-6 softmax and output. 256 columns of tensor memory and 112 KB of shared memory: two blocks per SM.
//   What was measured on the way (2,048 tokens, 32 heads on 2 kv heads, head_dim 128): P in tensor memory over its own
//   scores held a score buffer until the product P.V had read it, and the softmax threads stood idle four clocks in
//   ten waiting for the next scores; page ids read where they were needed and 2 KB copies (16 a tile) kept the producer
//   busy 1,000 clocks a tile. Two softmax threads a row (71 against 53 us), one block per SM with two tiles of 128
//   rows (67 us) and tiles of 128 keys with single-buffered scores (no gain) were slower or equal.
//
//   Pages past the entry's last page are read as the last page again (finite values the mask removes).
//   Every mbarrier wait is bounded; one that runs out sets *status and all roles leave their loops.
//
//   grid (tiles, kv heads). Tiles are numbered over the entries [first_entry, n_entries) in order; a block finds
//   its entry by walking entry_qstart.
#include "tcgen05.cuh"

#ifndef HEAD_DIM
#error "compile with -DHEAD_DIM=64 or 128"
#endif
static_assert(HEAD_DIM == 64 || HEAD_DIM == 128, "the tensor-memory prefill kernel takes head_dim 64 or 128");

constexpr int PT_HD = HEAD_DIM;
constexpr int PT_HALVES = HEAD_DIM / 64;          // 128-byte column blocks of a row
constexpr int PT_ROWS = 128;
constexpr int PT_KEYS = 64;
constexpr int PT_PAGE = 16;
constexpr int PT_TILE_PAGES = PT_KEYS / PT_PAGE;
constexpr int PT_K_STAGES = 2, PT_V_STAGES = 2;
constexpr int PT_Q_HALF = PT_ROWS * 128;          // bytes of one column block of Q
constexpr int PT_Q_BYTES = PT_HALVES * PT_Q_HALF;
constexpr int PT_P_BYTES = PT_ROWS * 128;         // P: 128 rows x 64 keys, bfloat16
constexpr int PT_ATOM = PT_HALVES * 1024;         // K and V tiles: 1 KB atoms (8 keys x 64 columns); a column block's atoms this far apart,
constexpr int PT_PAGE_BYTES = 2 * PT_ATOM;        // the next column block's 1 KB further; a page (16 keys) is two atoms of each
constexpr int PT_K_BYTES = PT_TILE_PAGES * PT_PAGE_BYTES;   // K tile; the V tile has the same size
constexpr int PT_THREADS = 224;
constexpr int PT_TMEM_COLS = 256;
constexpr int PT_COL_O = 2 * PT_KEYS;             // S buffers at columns 0 and 64, O behind them
constexpr int PT_N_BARS = 1 + 2 * PT_K_STAGES + 2 * PT_V_STAGES + 2 + 2 + 1 + 1;
// no slack for aligning the base: two blocks of head_dim 128 fill an SM's shared memory to within 2 KB; the base is checked instead
constexpr int PT_SMEM = PT_Q_BYTES + PT_P_BYTES + (PT_K_STAGES + PT_V_STAGES) * PT_K_BYTES + PT_N_BARS * 8 + 16;
constexpr unsigned PT_SPIN = 1u << 22;
constexpr float PT_RAISE = 8.f;                   // the running maximum follows a tile's only beyond this (log2 units)

// K or V of one page of one kv head (16 keys, all of head_dim) in one copy: the box of the cache's third tensor map
// (il_attn_decode_kv_map), which lands as [8 keys][column block][8 keys x 64 columns]: 1 KB atoms, interleaved by column block.
__device__ __forceinline__ void pt_tma_page(uint32_t dst, const CUtensorMap* map, int block16, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %3, %3, %3, %4}], [%2];\n"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(0), "r"(block16) : "memory");
}
__device__ __forceinline__ float pt_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pt_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(PT_THREADS, 2) attn_prefill_tc5_kernel(
    const __grid_constant__ CUtensorMap kv_map, const __nv_bfloat16* __restrict__ qkv, int row_stride,
    __nv_bfloat16* __restrict__ out, const int* __restrict__ block_table, int bt_stride, const int* __restrict__ entry_qstart,
    const int* __restrict__ entry_kvlen, int first_entry, int n_entries, int nh, int nkv, float scale_log2, int window, int tpt,
    int* __restrict__ status) {
    extern __shared__ __align__(1024) unsigned char smem[];
    if (t5_smem(smem) & 1023u) {                  // the swizzled tiles need 1 KB alignment; dynamic shared memory starts on it
        if (threadIdx.x == 0) atomicExch(status, 30);
        return;
    }
    const int G = nh / nkv;
    const int g = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // which entry and which tokens: tiles are taken from the last to the first, the longest blocks start first
    int tile = (int)gridDim.x - 1 - (int)blockIdx.x, e = first_entry;
    for (; e < n_entries; ++e) {
        const int nt = (entry_qstart[e + 1] - entry_qstart[e] + tpt - 1) / tpt;
        if (tile < nt) break;
        tile -= nt;
    }
    if (e >= n_entries) return;                   // the whole block
    const int q0 = entry_qstart[e], q1 = entry_qstart[e + 1];
    const int kvlen = entry_kvlen[e];
    const int start_pos = kvlen - (q1 - q0);
    const int tok0 = q0 + tile * tpt;
    const int n_tok = min(tpt, q1 - tok0);
    const int rows_valid = n_tok * G;
    const int* bt = block_table + (size_t)e * bt_stride;
    const int bpos_first = start_pos + (tok0 - q0), bpos_last = bpos_first + n_tok - 1;
    const int blo = (window > 0 && bpos_first - window + 1 > 0) ? bpos_first - window + 1 : 0;
    const int page_first = blo / PT_PAGE, page_last = bpos_last / PT_PAGE;
    const int n_tiles = (page_last - page_first) / PT_TILE_PAGES + 1;

    unsigned char* q_smem = smem;
    unsigned char* p_smem = smem + PT_Q_BYTES;
    unsigned char* k_smem = p_smem + PT_P_BYTES;
    unsigned char* v_smem = k_smem + PT_K_STAGES * PT_K_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(v_smem + PT_V_STAGES * PT_K_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + PT_N_BARS);
    const uint32_t bar0 = t5_smem(bars);
    const uint32_t q_full = bar0;                                     // Q is in shared memory (128 arrivals)
    const uint32_t k_full0 = bar0 + 8, k_empty0 = k_full0 + 8 * PT_K_STAGES;
    const uint32_t v_full0 = k_empty0 + 8 * PT_K_STAGES, v_empty0 = v_full0 + 8 * PT_V_STAGES;
    const uint32_t s_full0 = v_empty0 + 8 * PT_V_STAGES;              // a tile's scores are complete (tcgen05.commit)
    const uint32_t s_free0 = s_full0 + 16;                            // ... and read into registers: the buffer may be written again (4 warps)
    const uint32_t p_full = s_free0 + 16;                             // a tile's P is in shared memory (4 warps)
    const uint32_t o_done = p_full + 8;                               // a tile's P.V has been added to O, P may be written again (tcgen05.commit)

    if (threadIdx.x == 0) {
        t5_mbar_init(q_full, 128);
        for (int s = 0; s < PT_K_STAGES; ++s) {
            t5_mbar_init(k_full0 + 8 * s, 1);
            t5_mbar_init(k_empty0 + 8 * s, 1);
        }
        for (int s = 0; s < PT_V_STAGES; ++s) {
            t5_mbar_init(v_full0 + 8 * s, 1);
            t5_mbar_init(v_empty0 + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            t5_mbar_init(s_full0 + 8 * b, 1);
            t5_mbar_init(s_free0 + 8 * b, 4);
        }
        t5_mbar_init(p_full, 4);
        t5_mbar_init(o_done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    if (warp == 1) t5_alloc(tmem_slot, PT_TMEM_COLS);
    t5_fence_before();
    __syncthreads();
    t5_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- producer: K and V pages by TMA ----------------
        // One K or V tile: lane 0 waits for the slot, then one lane per page. Page ids come from the block table ahead of
        // their use: lane l holds the id of page base + l (`cur`) and of page base + 32 + l (`nxt`, still in flight when
        // it is loaded); a page's id is a shuffle away.
        int base = page_first;
        int cur = bt[min(base + lane, page_last)], nxt = bt[min(base + 32 + lane, page_last)];
        auto issue = [&](int j, int kv) -> bool {
            const int stage = kv ? j % PT_V_STAGES : j % PT_K_STAGES, round = kv ? j / PT_V_STAGES : j / PT_K_STAGES;
            const uint32_t full = (kv ? v_full0 : k_full0) + 8 * stage;
            while (kv && page_first + j * PT_TILE_PAGES >= base + 32) {   // V(j) is the tile furthest behind: the window follows it
                base += 32;
                cur = nxt;
                nxt = bt[min(base + 32 + lane, page_last)];
            }
            int ok = 1;
            if (lane == 0) {
                if (!t5_mbar_wait((kv ? v_empty0 : k_empty0) + 8 * stage, ((uint32_t)round & 1u) ^ 1u, PT_SPIN)) {
                    atomicExch(status, 31);
                    ok = 0;
                } else {
                    t5_mbar_expect_tx(full, PT_K_BYTES);
                }
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            const int p = lane % PT_TILE_PAGES;
            const int off = min(page_first + j * PT_TILE_PAGES + p, page_last) - base;      // 0 .. 63: K runs ahead of V
            const int id_cur = __shfl_sync(0xffffffffu, cur, off & 31), id_nxt = __shfl_sync(0xffffffffu, nxt, off & 31);
            if (ok && lane < PT_TILE_PAGES) {
                const int page = off < 32 ? id_cur : id_nxt;
                const uint32_t dst = t5_smem((kv ? v_smem : k_smem) + stage * PT_K_BYTES + p * PT_PAGE_BYTES);
                pt_tma_page(dst, &kv_map, (page * 2 + kv) * nkv + g, full);
            }
            return ok != 0;
        };
        // K runs up to two tiles ahead (its slots are free once the scores are computed), V follows the products
        bool ok = issue(0, 0);
        if (ok && n_tiles > 1) ok = issue(1, 0);
        for (int j = 0; j < n_tiles && ok; ++j) {
            ok = issue(j, 1);
            if (ok && j + 2 < n_tiles) ok = issue(j + 2, 0);
        }
    } else if (warp == 1) {
        // ---------------- tensor-core issue, scores: S(j) as soon as K(j) is there and the buffer has been read out ----------------
        // Two issuing threads, one for each kind of product: a wait on an mbarrier costs the thread about 200 clocks
        // even when it is over already, and one thread with four of them a tile was what a tile's time came to.
        if (lane == 0) {
            // The issuing thread must keep up with the tensor core (a product every 32 to 64 clocks), so every descriptor
            // is made here, once: per product only an add of a constant remains. In a descriptor the address field counts
            // 16-byte units: 32 bytes along K inside the swizzle span are +2.
            const uint32_t idesc_s = t5_idesc(PT_ROWS, PT_KEYS, false);
            const uint64_t q_desc = t5_desc(t5_smem(q_smem), 16, 1024);
            const uint64_t k_desc0 = t5_desc(t5_smem(k_smem), 16, PT_ATOM);                // slot s: + s * slot bytes / 16
            bool ok = t5_mbar_wait(q_full, 0, PT_SPIN);
            if (!ok) atomicExch(status, 32);
            for (int j = 0; j < n_tiles && ok; ++j) {
                const int s = j % PT_K_STAGES, b = j & 1;
                if (!t5_mbar_wait(k_full0 + 8 * s, (uint32_t)(j / PT_K_STAGES) & 1u, PT_SPIN)) { atomicExch(status, 35); ok = false; break; }
                // the score buffer: read out by the softmax of tile j-2 (nothing to wait for on a buffer's first use)
                if (j >= 2 && !t5_mbar_wait(s_free0 + 8 * b, (uint32_t)((j >> 1) - 1) & 1u, PT_SPIN)) { atomicExch(status, 39); ok = false; break; }
                t5_fence_after();
                const uint64_t kd = k_desc0 + (uint64_t)(s * (PT_K_BYTES >> 4));
                const uint32_t s_tmem = tmem_base + (uint32_t)(b * PT_KEYS);
#pragma unroll
                for (int kk = 0; kk < PT_HD / 16; ++kk) {
                    const uint64_t off_q = (uint64_t)((kk >> 2) * (PT_Q_HALF >> 4) + (kk & 3) * 2);
                    const uint64_t off_k = (uint64_t)((kk >> 2) * (1024 >> 4) + (kk & 3) * 2);
                    t5_mma_ss(s_tmem, q_desc + off_q, kd + off_k, idesc_s, kk > 0 ? 1u : 0u);
                }
                t5_commit(s_full0 + 8 * b);
                t5_commit(k_empty0 + 8 * s);                  // and the K slot is free
            }
        }
    } else if (warp == 2) {
        // ---------------- tensor-core issue, outputs: O += P.V(j) as soon as P(j) and V(j) are there ----------------
        if (lane == 0) {
            const uint32_t idesc_o = t5_idesc(PT_ROWS, PT_HD, true);
            const uint64_t p_desc = t5_desc(t5_smem(p_smem), 16, 1024);
            const uint64_t v_desc0 = t5_desc(t5_smem(v_smem), 1024, PT_ATOM);
            const uint32_t o_tmem = tmem_base + PT_COL_O;
            for (int i = 0; i < n_tiles; ++i) {
                const int s = i % PT_V_STAGES;
                if (!t5_mbar_wait(v_full0 + 8 * s, (uint32_t)(i / PT_V_STAGES) & 1u, PT_SPIN)) { atomicExch(status, 34); break; }
                if (!t5_mbar_wait(p_full, (uint32_t)i & 1u, PT_SPIN)) { atomicExch(status, 33); break; }
                t5_fence_after();
                const uint64_t vd = v_desc0 + (uint64_t)(s * (PT_K_BYTES >> 4));
#pragma unroll
                for (int kk = 0; kk < PT_KEYS / 16; ++kk)     // 16 keys a product: 32 bytes along a row of P, one page of V
                    t5_mma_ss(o_tmem, p_desc + (uint64_t)(kk * 2), vd + (uint64_t)(kk * (PT_PAGE_BYTES >> 4)), idesc_o, (i > 0 || kk > 0) ? 1u : 0u);
                t5_commit(v_empty0 + 8 * s);                  // the V slot is free once these products have read it
                t5_commit(o_done);                            // and so is P's place
            }
        }
    } else {
        // ---------------- softmax and output: warps 3..6 own tensor-memory lanes 32*(warp % 4) .. +31 ----------------
        const int qd = warp & 3;
        const int r = qd * 32 + lane;                         // this thread's row
        const bool rvalid = r < rows_valid;
        const int tl = rvalid ? r / G : 0, hh = rvalid ? r - tl * G : 0;
        const int rpos = rvalid ? bpos_first + tl : -1;       // a row that is not there masks every key
        const int rlo = (rvalid && window > 0 && rpos - window + 1 > 0) ? rpos - window + 1 : 0;
        {   // Q: this row's head_dim values into the swizzled K-major tile (16-byte chunk c of row r at chunk c ^ (r % 8))
            const uint4* src = rvalid ? reinterpret_cast<const uint4*>(qkv + (size_t)(tok0 + tl) * row_stride + (size_t)(g * G + hh) * PT_HD) : nullptr;
#pragma unroll
            for (int kk = 0; kk < PT_HALVES; ++kk)
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const uint4 v = src ? src[kk * 8 + c] : make_uint4(0u, 0u, 0u, 0u);
                    *reinterpret_cast<uint4*>(q_smem + kk * PT_Q_HALF + r * 128 + ((c ^ (r & 7)) << 4)) = v;
                }
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");      // the tensor core reads it through the async proxy
            t5_mbar_arrive(q_full);
        }
        const uint32_t t_lane = tmem_base + ((uint32_t)(qd * 32) << 16);
        unsigned char* p_row = p_smem + r * 128;
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < n_tiles; ++j) {
            const int b = j & 1;
            if (!t5_mbar_wait(s_full0 + 8 * b, (uint32_t)(j >> 1) & 1u, PT_SPIN)) { atomicExch(status, 36); ok = false; break; }
            t5_fence_after();
            uint32_t sv[PT_KEYS];
            t5_ld32(t_lane + b * PT_KEYS, sv);
            t5_ld32(t_lane + b * PT_KEYS + 32, sv + 32);
            t5_wait_ld();
            // the scores are in registers: the tensor core may write this buffer again (tile j+2)
            t5_fence_before();
            __syncwarp();
            if (lane == 0) t5_mbar_arrive(s_free0 + 8 * b);
            const int kb = (page_first + j * PT_TILE_PAGES) * PT_PAGE;
            if (kb + PT_KEYS - 1 > rpos || kb < rlo) {        // the tile touches this row's causal or window edge
#pragma unroll
                for (int c = 0; c < PT_KEYS; ++c) {
                    const int key = kb + c;
                    if (!(key <= rpos && key >= rlo)) sv[c] = __float_as_uint(-INFINITY);
                }
            }
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};      // four chains: a single one is all latency
#pragma unroll
            for (int c = 0; c < PT_KEYS; c += 4)
#pragma unroll
                for (int i = 0; i < 4; ++i) mx4[i] = fmaxf(mx4[i], __uint_as_float(sv[c + i]));
            const float mxs = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;      // scale > 0
            const bool raise = mxs > m + PT_RAISE;            // also the first keys a row sees (m = -inf)
            const float m_new = raise ? mxs : m;
            const float corr = raise ? pt_ex2(m - m_new) : 1.f;   // 0 when nothing was summed yet
            const float msafe = (m_new == -INFINITY) ? 0.f : m_new;
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int c = 0; c < PT_KEYS; c += 2) {
                const float a = pt_ex2(fmaf(__uint_as_float(sv[c]), scale_log2, -msafe));
                const float bb = pt_ex2(fmaf(__uint_as_float(sv[c + 1]), scale_log2, -msafe));
                sum4[(c >> 1) & 3] += a + bb;
                sv[c >> 1] = pt_pack(a, bb);
            }
            l = l * corr + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
            m = m_new;
            if (j > 0) {
                // P's place in shared memory is free, and O holds the tiles before this one, only when their last product is through
                if (!t5_mbar_wait(o_done, (uint32_t)(j - 1) & 1u, PT_SPIN)) { atomicExch(status, 37); ok = false; break; }
                t5_fence_after();
                if (__any_sync(0xffffffffu, raise)) {
#pragma unroll
                    for (int c0 = 0; c0 < PT_HD; c0 += 32) {
                        uint32_t ov[32];
                        t5_ld32(t_lane + PT_COL_O + c0, ov);
                        t5_wait_ld();
#pragma unroll
                        for (int c = 0; c < 32; ++c) ov[c] = __float_as_uint(__uint_as_float(ov[c]) * corr);
                        t5_st32(t_lane + PT_COL_O + c0, ov);
                    }
                    t5_wait_st();
                }
            }
            // P: this row's 64 values as 8 chunks of 16 bytes of the swizzled K-major tile
#pragma unroll
            for (int c = 0; c < 8; ++c)
                *reinterpret_cast<uint4*>(p_row + ((c ^ (r & 7)) << 4)) = make_uint4(sv[4 * c], sv[4 * c + 1], sv[4 * c + 2], sv[4 * c + 3]);
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            t5_fence_before();
            __syncwarp();
            if (lane == 0) t5_mbar_arrive(p_full);
        }
        if (ok) {
            if (!t5_mbar_wait(o_done, (uint32_t)(n_tiles - 1) & 1u, PT_SPIN)) {
                atomicExch(status, 38);
            } else {
                t5_fence_after();
                const float inv = (l > 0.f) ? 1.f / l : 0.f;
                // The rows go out through shared memory (Q's place: every product that reads Q is through): a thread owns a
                // row of tensor memory, but 16-byte stores 8 KB apart cost a block 2 us; a warp's 32 rows are stored
                // 32 / CH at a time instead, CH lanes a row, each row's bytes contiguous.
                constexpr int CH = PT_HD / 8;                 // 16-byte chunks of a row
                unsigned char* stage = q_smem + qd * 32 * (PT_HD * 2);
#pragma unroll
                for (int c0 = 0; c0 < PT_HD; c0 += 32) {
                    uint32_t ov[32];
                    t5_ld32(t_lane + PT_COL_O + c0, ov);
                    t5_wait_ld();
#pragma unroll
                    for (int c = 0; c < 32; c += 8) {
                        uint4 v;
                        v.x = pt_pack(__uint_as_float(ov[c]) * inv, __uint_as_float(ov[c + 1]) * inv);
                        v.y = pt_pack(__uint_as_float(ov[c + 2]) * inv, __uint_as_float(ov[c + 3]) * inv);
                        v.z = pt_pack(__uint_as_float(ov[c + 4]) * inv, __uint_as_float(ov[c + 5]) * inv);
                        v.w = pt_pack(__uint_as_float(ov[c + 6]) * inv, __uint_as_float(ov[c + 7]) * inv);
                        const int ch = (c0 + c) >> 3;
                        *reinterpret_cast<uint4*>(stage + lane * (PT_HD * 2) + ((ch ^ (lane & 7)) << 4)) = v;
                    }
                }
                __syncwarp();
#pragma unroll
                for (int it = 0; it < CH; ++it) {
                    const int wr = it * (32 / CH) + lane / CH, ch = lane % CH;      // row of this warp, chunk of the row
                    const int rr = qd * 32 + wr;
                    if (rr < rows_valid) {
                        const int t2 = rr / G, h2 = rr - t2 * G;
                        const uint4 v = *reinterpret_cast<const uint4*>(stage + wr * (PT_HD * 2) + ((ch ^ (wr & 7)) << 4));
                        *reinterpret_cast<uint4*>(out + (size_t)(tok0 + t2) * nh * PT_HD + (size_t)(g * G + h2) * PT_HD + ch * 8) = v;
                    }
                }
            }
        }
    }
    t5_fence_before();
    __syncthreads();
    if (warp == 1) {
        t5_fence_after();
        t5_dealloc(tmem_base, PT_TMEM_COLS);
    }
}

// Rows a block owns: it takes rows / (heads per kv head) consecutive tokens.
IL_EXPORT int il_attn_prefill_tc5_rows() { return PT_ROWS; }

// kv_map: the 128 bytes of the cache's third tensor map (il_attn_decode_kv_map: a page's K or V as tensor-core tiles), on the host.
// n_tiles_total: sum over entries [first_entry, n_entries) of ceil(q_len / tpt), tpt = max(1, rows / (nh/nkv)), rows = il_attn_prefill_tc5_rows().
IL_EXPORT int il_attn_prefill_tc5(const void* qkv, int row_stride, void* out, const void* kv_map, const int* block_table,
                                  int bt_stride, const int* entry_qstart, const int* entry_kvlen, int page_size, int first_entry,
                                  int n_entries, int n_tiles_total, int nh, int nkv, int hd, float scale, int window, int* status,
                                  cudaStream_t stream) {
    if (n_tiles_total <= 0 || first_entry >= n_entries) return IL_OK;
    if (hd != HEAD_DIM || page_size != PT_PAGE || !kv_map || !status) return IL_UNSUPPORTED;
    if (nh <= 0 || nkv <= 0 || nh % nkv != 0) return IL_BAD_ARG;
    const int G = nh / nkv;
    if (G > PT_ROWS || scale <= 0.f) return IL_UNSUPPORTED;
    if (((uintptr_t)qkv & 15) || ((uintptr_t)out & 15) || (row_stride & 7)) return IL_UNSUPPORTED;
    int dev = 0;
    cudaGetDevice(&dev);
    static bool attr_set[64];
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PT_SMEM);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(attn_prefill_tc5_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return 1000 + (int)e;
        attr_set[dev] = true;
    }
    CUtensorMap map;
    memcpy(&map, kv_map, sizeof(map));
    dim3 grid(n_tiles_total, nkv);
    attn_prefill_tc5_kernel<<<grid, PT_THREADS, PT_SMEM, stream>>>(
        map, (const __nv_bfloat16*)qkv, row_stride, (__nv_bfloat16*)out, block_table, bt_stride, entry_qstart, entry_kvlen,
        first_entry, n_entries, nh, nkv, scale * 1.4426950408889634f, window, PT_ROWS / G, status);
    IL_LAUNCH_CHECK();
    return IL_OK;
}
