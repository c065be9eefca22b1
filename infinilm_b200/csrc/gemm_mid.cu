// Matrix products for 17..128 activation rows (decode at large batch, short prompt portions) on the 5th-generation
// tensor cores, with what follows a projection in a decoder layer done in the epilogue:
//     plain     out[M,N] = alpha * x[M,K] . W[N,K]^T (+ bias)
//     SwiGLU    out[M,N] = silu(alpha * x . Wg^T + bg) * (alpha * x . Wu^T + bu),  W = [Wg; Wu]
//
//   The weights are the A operand: a tile is 64 rows of W (tcgen05.mma with M = 64, whose accumulator row r lies in lane
//   32 * (r / 16) + r % 16 of tensor memory), x is the B operand in blocks of NB activation rows, and a unit of work is
//   one tile x one block of activation rows over ALL of K. Nothing is cut along K, so no partial sums pass between
//   blocks: every attempt to cut along K here lost more at the end of the kernel, where the parts meet, than the even
//   shares had gained. A tile's weights are read once from memory and again from L2 by the units of the other row
//   blocks, which are numbered next to it and so run at the same time on other SMs.
//   The SwiGLU form keeps two accumulators per unit, gate rows and the up rows that go with them, in the same lanes.
//
//   Blocks are persistent (one per SM) and take units b, b + G, ... Roles by warp: warp 0 issues TMA tensor copies
//   (128-byte swizzle) into a ring of stages - the first ring of weight tiles before the dependent-launch wait, since
//   weights do not come from the kernel before -, warps 1-4 issue tcgen05.mma (two or four of them), each into an accumulator
//   of its own, and commit (two accumulator sets alternate, so a unit's epilogue overlaps the next unit's products), warps 5-8
//   read their lanes of tensor memory and finish.
//
//   Every mbarrier wait is bounded; one that runs out sets *status, the roles leave their loops, the block frees its
//   tensor memory and returns.
#include <cuda.h>

#include "common.cuh"

constexpr int GM_BK = 64;                         // K per tensor copy: 128 bytes, the swizzle span
constexpr int GM_KBLK = 4;                        // copies (of each operand) per stage, at most: the issuing thread pays some 400 clocks
                                                  // per stage for its wait and commit, which 12 KB a stage did not cover (20 GB/s an SM)
constexpr int GM_MAX_STAGES = 6;
constexpr int GM_THREADS = 288;                   // producer, up to four issuers, four epilogue warps
constexpr int GM_MAX_ROWS = 128;
constexpr unsigned GM_SPIN_LIMIT = 1u << 26;

__device__ __forceinline__ uint32_t gm_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void gm_mbar_init(uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void gm_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void gm_mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool gm_mbar_wait(uint32_t bar, uint32_t parity) {
    for (unsigned spin = 0; spin < GM_SPIN_LIMIT; ++spin) {
        uint32_t done;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void gm_tma_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];\n"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void gm_tma_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
// Shared-memory matrix descriptor, K-major, 128-byte swizzle: 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t gm_desc(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFF) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}
__device__ __forceinline__ void gm_mma(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}\n"
                 ::"r"(d_tmem), "l"(a), "l"(b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void gm_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void gm_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                   "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
}

enum { GM_PLAIN = 0, GM_GLU = 1 };


struct GmParams {
    int M, N, K;                                  // N: output columns (SwiGLU: the intermediate size; W has 2N rows)
    int mode, n_acc;                              // accumulators per unit: 1 plain, 2 SwiGLU (gate, up)
    int NB, n_bb;                                 // activation rows per unit (a multiple of 16), blocks of them
    int n_issuers;                                // threads that issue products, each into an accumulator of its own
    int tma3d;                                    // the tensor maps are the three-dimensional ones (K a multiple of 64)
    int n_tiles, n_chunks, n_stages, n_units, kblk, bm;   // kblk: 64-wide blocks of K per stage; bm: W rows per tile
    int ldo, out_kind;
    float alpha;
    const float* bias;                            // [N], SwiGLU [2N], or null
    void* out;
    int* status;
};

// KB: 64-wide blocks of K per stage; NACC: accumulators per unit. Both are template arguments so that the thread that
// issues the products runs a flat list of instructions: with loops and descriptors worked out per product it spent some
// hundred clocks on each, and a product of M = 64 covers only 2 KB of weights - 40 GB/s an SM, half of what is needed.
// BM: W rows per accumulator (the MMA's M), 64 or 128.
template <int KB, int NACC, int BM>
__global__ void __launch_bounds__(GM_THREADS, 1) gemm_mid_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                 const __grid_constant__ CUtensorMap map_w2,
                                                                 const __grid_constant__ CUtensorMap map_x, const GmParams p) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int GM_BM = BM;
    const int a_bytes = GM_BM * GM_BK * 2, b_bytes = p.NB * GM_BK * 2;    // one 64-wide block of K of each operand
    constexpr int n_a = NACC;
    const int stage_bytes = KB * (n_a * a_bytes + b_bytes);               // [accumulator][k block] weights, then [k block] activations
    const int STAGES = p.n_stages;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * stage_bytes);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * GM_MAX_STAGES + 4);
    const uint32_t full0 = gm_smem(bars), empty0 = full0 + GM_MAX_STAGES * 8;
    const uint32_t tfull0 = empty0 + GM_MAX_STAGES * 8, tempty0 = tfull0 + 2 * 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = gridDim.x, b = blockIdx.x;
    const int NI = p.n_issuers;                   // issuing threads: 2, or 4 (plain products with four blocks of K per stage)
    const int acc_cols = NI * p.NB;               // tensor-memory columns of one accumulator set: an accumulator per issuer
    uint32_t ncols = 32;
    while ((int)ncols < 2 * acc_cols) ncols <<= 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            gm_mbar_init(full0 + s * 8, 1);
            gm_mbar_init(empty0 + s * 8, NI);     // every issuer
        }
        for (int a = 0; a < 2; ++a) {
            gm_mbar_init(tfull0 + a * 8, NI);
            gm_mbar_init(tempty0 + a * 8, 4);     // one arrival per epilogue warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(gm_smem(tmem_slot)), "r"(ncols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    // unit u -> (tile, block of activation rows); the row blocks of a tile are neighbours in u
    const int n_my = b < p.n_units ? (p.n_units - b + G - 1) / G : 0;
    const long long total = (long long)n_my * p.n_chunks;     // (unit, chunk) pairs of this block, in order

    if (warp == 0) {
        // ---------------- producer ----------------
        if (lane == 0) {
            auto issue = [&](int tile, int bb, int c, int stage, bool weights, bool acts) {
                const uint32_t full = full0 + stage * 8, dst = gm_smem(smem + stage * stage_bytes);
                if (weights) gm_mbar_expect_tx(full, (uint32_t)stage_bytes);
                if (p.tma3d) {
                    // K a multiple of 64: the operands are seen as [K / 64][rows][64] and all the stage's blocks of K of an
                    // operand come in one copy (a copy costs its issuing thread some 100 clocks)
                    if (weights) {
                        gm_tma_3d(dst, &map_w, 0, tile * GM_BM, c * KB, full);
                        if (n_a == 2) gm_tma_3d(dst + KB * a_bytes, &map_w2, 0, tile * GM_BM, c * KB, full);
                    }
                    if (acts) gm_tma_3d(dst + KB * n_a * a_bytes, &map_x, 0, bb * p.NB, c * KB, full);
                } else {
                    if (weights) {
                        for (int kb = 0; kb < KB; ++kb) {         // blocks past the end of K come in as zeros
                            gm_tma_2d(dst + kb * a_bytes, &map_w, (c * KB + kb) * GM_BK, tile * GM_BM, full);
                            if (n_a == 2) gm_tma_2d(dst + (KB + kb) * a_bytes, &map_w2, (c * KB + kb) * GM_BK, tile * GM_BM, full);
                        }
                    }
                    if (acts) {
                        for (int kb = 0; kb < KB; ++kb)
                            gm_tma_2d(dst + KB * n_a * a_bytes + kb * b_bytes, &map_x, (c * KB + kb) * GM_BK, bb * p.NB, full);
                    }
                }
            };
            // (unit, chunk) pairs in order, without a division per pair: k counts this block's units, c the chunks of K
            const int n_early = (int)(total < STAGES ? total : STAGES);
            {
                int k = 0, c = 0;
                for (int i = 0; i < n_early; ++i) {               // the ring is empty: no wait; weights only
                    const int u = b + k * G, tile = u / p.n_bb;
                    issue(tile, u - tile * p.n_bb, c, i, true, false);
                    if (++c == p.n_chunks) { c = 0; ++k; }
                }
            }
            il_pdl_wait();                        // x comes from the kernel before
            int k = 0, c = 0;
            for (int i = 0; i < n_early; ++i) {
                const int u = b + k * G, tile = u / p.n_bb;
                issue(tile, u - tile * p.n_bb, c, i, false, true);
                if (++c == p.n_chunks) { c = 0; ++k; }
            }
            int stage = n_early == STAGES ? 0 : n_early;
            uint32_t phase = n_early == STAGES ? 1 : 0;
            for (; k < n_my; ++k, c = 0) {
                const int u = b + k * G, tile = u / p.n_bb, bb = u - tile * p.n_bb;
                bool ok = true;
                for (; c < p.n_chunks; ++c) {
                    if (!gm_mbar_wait(empty0 + stage * 8, phase ^ 1)) { atomicExch(p.status, 51); ok = false; break; }
                    issue(tile, bb, c, stage, true, true);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
            }
        }
    } else if (warp >= 1 && warp <= 4) {
        // ---------------- tensor-core issue: two threads, each with an accumulator of its own ----------------
        // Every issuer has an accumulator of its own. SwiGLU: gate (issuer 0) and up (issuer 1). Plain: the stage's 64-wide
        // blocks of K dealt out in turn to two or four issuers; the epilogue adds their accumulators. One thread issues a
        // product every 55 clocks at best (measured on fixed operands; 76 in this loop) and a product of M = 64 covers
        // only 2 KB of weights, which is half of what the memory's rate needs; the tensor pipe itself takes some 25 clocks
        // for such a product when several threads feed it.
        if (lane == 0 && warp - 1 < NI) {
            const int me = warp - 1;
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(p.NB >> 3) << 17) | ((uint32_t)(GM_BM >> 4) << 24);
            int stage = 0, acc = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            for (int k = 0; k < n_my && ok; ++k) {
                if (!gm_mbar_wait(tempty0 + acc * 8, acc_phase ^ 1)) { atomicExch(p.status, 52); break; }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * acc_cols + me * p.NB);
                for (int c = 0; c < p.n_chunks; ++c) {
                    if (!gm_mbar_wait(full0 + stage * 8, phase)) { atomicExch(p.status, 53); ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    const uint32_t sa = gm_smem(smem + stage * stage_bytes);
                    // descriptors count addresses in 16-byte units in their low bits: the next operand block is an addition
                    const uint64_t da0 = gm_desc(sa), db0 = gm_desc(sa + KB * n_a * a_bytes);
                    const uint64_t b_step = (uint64_t)(b_bytes >> 4);
                    if (NACC == 2) {
#pragma unroll
                        for (int kb = 0; kb < KB; ++kb)
#pragma unroll
                            for (int kk = 0; kk < GM_BK / 16; ++kk)   // 32 bytes further along K inside the swizzle span
                                gm_mma(d_tmem, da0 + (uint64_t)(((me * KB + kb) * a_bytes >> 4) + kk * 2),
                                       db0 + (uint64_t)kb * b_step + (uint64_t)(kk * 2), idesc, (c > 0 || kb > 0 || kk > 0) ? 1u : 0u);
                    } else {
                        for (int kb = me; kb < KB; kb += NI) {        // this issuer's blocks of K
#pragma unroll
                            for (int kk = 0; kk < GM_BK / 16; ++kk)
                                gm_mma(d_tmem, da0 + (uint64_t)((kb * a_bytes >> 4) + kk * 2), db0 + (uint64_t)kb * b_step + (uint64_t)(kk * 2),
                                       idesc, (c > 0 || kb > me || kk > 0) ? 1u : 0u);
                        }
                    }
                    gm_commit(empty0 + stage * 8);            // the stage is free once both issuers' products have read it
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                gm_commit(tfull0 + acc * 8);                  // this issuer's accumulator is complete
                if (++acc == 2) { acc = 0; acc_phase ^= 1; }
            }
        }
    } else if (warp >= 5) {
        // ---------------- epilogue: warp w reads tensor-memory lanes 32 * (w % 4) .. + 31, of which the first 16 hold
        // rows 16 * (w % 4) .. + 15 of the tile ----------------
        il_pdl_wait();                            // these warps write the output
        const int q = warp & 3;                   // warps 5..8
        const bool live = BM == 128 || lane < 16;
        const int row = BM == 128 ? q * 32 + lane : q * 16 + lane;    // this thread's W row within the tile (M = 64: lanes 16..31 have none)
        int acc = 0;
        uint32_t acc_phase = 0;
        for (int k = 0; k < n_my; ++k) {
            const int u = b + k * G, tile = u / p.n_bb, bb = u - tile * p.n_bb;
            if (!gm_mbar_wait(tfull0 + acc * 8, acc_phase)) { if (lane == 0) atomicExch(p.status, 54); break; }
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * acc_cols);
            const int n = tile * GM_BM + row, m0 = bb * p.NB;
            const bool n_ok = live && n < p.N;
            const float bg = (p.bias && n_ok) ? p.bias[n] : 0.f;
            const float bu = (p.mode == GM_GLU && p.bias && n_ok) ? p.bias[p.N + n] : 0.f;
            for (int j0 = 0; j0 < p.NB; j0 += 16) {
                uint32_t vg[16], vu[16];
                gm_ld16(taddr + j0, vg);
                gm_ld16(taddr + p.NB + j0, vu);
                asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                float y[16];
                if (p.mode == GM_GLU) {
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        y[j] = il_silu_mul_fast(__fmaf_rn(p.alpha, __uint_as_float(vg[j]), bg), __fmaf_rn(p.alpha, __uint_as_float(vu[j]), bu));
                } else {                          // the issuers' shares of K, added in the order of the issuers
                    float sum[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) sum[j] = __uint_as_float(vg[j]) + __uint_as_float(vu[j]);
                    if (NI == 4) {
                        gm_ld16(taddr + 2 * p.NB + j0, vg);
                        gm_ld16(taddr + 3 * p.NB + j0, vu);
                        asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
                        for (int j = 0; j < 16; ++j) sum[j] = (sum[j] + __uint_as_float(vg[j])) + __uint_as_float(vu[j]);
                    }
#pragma unroll
                    for (int j = 0; j < 16; ++j) y[j] = __fmaf_rn(p.alpha, sum[j], bg);
                }
                if (n_ok) {
                    if (p.out_kind == IL_F32) {
                        float* o = (float*)p.out + (size_t)(m0 + j0) * p.ldo + n;
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (m0 + j0 + j < p.M) o[(size_t)j * p.ldo] = y[j];
                    } else {
                        __nv_bfloat16* o = (__nv_bfloat16*)p.out + (size_t)(m0 + j0) * p.ldo + n;
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (m0 + j0 + j < p.M) o[(size_t)j * p.ldo] = __float2bfloat16_rn(y[j]);
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) gm_mbar_arrive(tempty0 + acc * 8);
            if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
    }
    il_pdl_tail();
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(ncols) : "memory");
    }
}

typedef CUresult (*gm_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static gm_encode_fn gm_encoder() {
    static gm_encode_fn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (gm_encode_fn)p;
    }
    return fn;
}

// A [rows x K] bfloat16 matrix with row stride ld, read in boxes of [box_rows x 64] with the 128-byte swizzle.
static int gm_make_map(CUtensorMap* map, const void* base, int rows, int K, int ld, int box_rows) {
    gm_encode_fn enc = gm_encoder();
    if (!enc) return IL_UNSUPPORTED;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)GM_BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 2000 + (int)r;
}

// The same matrix as [K / 64][rows][64] (K a multiple of 64), read in boxes of [kblk][box_rows][64]: kblk blocks of K at once,
// each landing as a [box_rows x 64] tile with the 128-byte swizzle.
static int gm_make_map3(CUtensorMap* map, const void* base, int rows, int K, int ld, int box_rows, int kblk) {
    gm_encode_fn enc = gm_encoder();
    if (!enc) return IL_UNSUPPORTED;
    cuuint64_t dims[3] = {(cuuint64_t)GM_BK, (cuuint64_t)rows, (cuuint64_t)(K / GM_BK)};
    cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)GM_BK * 2};
    cuuint32_t box[3] = {(cuuint32_t)GM_BK, (cuuint32_t)box_rows, (cuuint32_t)kblk};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 2000 + (int)r;
}

static int gm_sm_count() {
    static int n[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return 1;
    if (!n[dev] && (cudaDeviceGetAttribute(&n[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n[dev] <= 0)) n[dev] = 1;
    return n[dev];
}

// Activation rows per unit: the largest block (a multiple of 16 up to the padded row count) that still gives (nearly)
// every SM a unit; more, smaller blocks only re-read the weights from L2 more often.
static int gm_pick_nb(int Mp, int n_tiles, int n_sm) {
    int best = 16;
    for (int nb = 16; nb <= Mp; nb += 16) {
        const int n_bb = (Mp + nb - 1) / nb;
        if (n_bb * nb - Mp >= 16) continue;       // a block of padding only
        if ((long long)n_tiles * n_bb * 100 >= (long long)n_sm * 85 || nb == 16) best = nb;
    }
    return best;
}

IL_EXPORT int il_gemm_mid_max_rows() { return GM_MAX_ROWS; }

// glu = 1: W is [2N, K] (N gate rows, then N up rows), bias [2N], out[M,N] = silu(alpha*x.Wg^T + bg) * (alpha*x.Wu^T + bu).
// nb: activation rows per unit, bm_want: weight rows per tile, 64 or 128 (0: chosen here).
IL_EXPORT int il_gemm_mid(const void* x, int ldx, const void* W, int ldw, void* out, int out_kind, int ldo, const float* bias,
                          float alpha, int M, int N, int K, int glu, int nb, int bm_want, int* status, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return IL_OK;
    if (M > GM_MAX_ROWS || K <= 0 || (K & 7) || (ldx & 7) || (ldw & 7) || ldx < K || ldw < K || ldo < N || !status) return IL_UNSUPPORTED;
    if (((uintptr_t)x & 15) || ((uintptr_t)W & 15)) return IL_UNSUPPORTED;
    if (out_kind != IL_F32 && out_kind != IL_BF16) return IL_BAD_ARG;
    if (glu && out_kind != IL_BF16) return IL_UNSUPPORTED;
    const int n_sm = gm_sm_count();
    const int Mp = (M + 15) & ~15;

    GmParams p;
    p.M = M; p.N = N; p.K = K; p.mode = glu ? GM_GLU : GM_PLAIN; p.n_acc = glu ? 2 : 1;
    // tiles of 128 rows where that still gives (nearly) every SM a unit at whole activation blocks: a product of M = 64
    // covers 2 KB of weights and the tensor pipe takes some 80 clocks for it, which holds an SM to about 50 GB/s
    const int bm = bm_want > 0 ? bm_want : ((long long)((N + 127) / 128) * 100 >= (long long)n_sm * 85 ? 128 : 64);
    if (bm != 64 && bm != 128) return IL_BAD_ARG;
    p.bm = bm;
    p.n_tiles = (N + bm - 1) / bm;

    p.NB = nb > 0 ? nb : gm_pick_nb(Mp, p.n_tiles, n_sm);
    if (p.NB % 16 || p.NB < 16 || p.NB > 128) return IL_BAD_ARG;
    p.n_bb = (Mp + p.NB - 1) / p.NB;
    p.n_units = p.n_tiles * p.n_bb;
    p.ldo = ldo; p.out_kind = out_kind; p.alpha = alpha; p.bias = bias; p.out = out; p.status = status;

    const int a_bytes = bm * GM_BK * 2, b_bytes = p.NB * GM_BK * 2;
    const int tail = (2 * GM_MAX_STAGES + 4) * 8 + 16;
    int kblk = GM_KBLK, stage_bytes = 0, n_stages = 0;
    for (;; kblk >>= 1) {                         // as much of K per stage as leaves a ring of at least three stages
        stage_bytes = kblk * (p.n_acc * a_bytes + b_bytes);
        n_stages = (227 * 1024 - 1024 - tail) / stage_bytes;
        if (n_stages >= 4 || kblk == (glu ? 1 : 2)) break;
    }
    if (n_stages > GM_MAX_STAGES) n_stages = GM_MAX_STAGES;
    if (n_stages < 2) return IL_UNSUPPORTED;
    p.n_stages = n_stages;
    p.kblk = kblk;
    p.n_issuers = (!glu && kblk == 4 && p.NB <= 64) ? 4 : 2;      // (four accumulators of NB columns, twice, must fit 512 columns)
    p.n_chunks = (K + GM_BK * kblk - 1) / (GM_BK * kblk);
    p.tma3d = (K % GM_BK == 0) ? 1 : 0;

    CUtensorMap map_w, map_w2, map_x;
    int rc;
    if (p.tma3d) {
        rc = gm_make_map3(&map_w, W, N, K, ldw, bm, kblk);
        if (rc) return rc;
        map_w2 = map_w;
        if (glu) rc = gm_make_map3(&map_w2, (const __nv_bfloat16*)W + (size_t)N * ldw, N, K, ldw, bm, kblk);
        if (rc) return rc;
        rc = gm_make_map3(&map_x, x, M, K, ldx, p.NB, kblk);
        if (rc) return rc;
    } else {
        rc = gm_make_map(&map_w, W, N, K, ldw, bm);
        if (rc) return rc;
        map_w2 = map_w;
        if (glu) rc = gm_make_map(&map_w2, (const __nv_bfloat16*)W + (size_t)N * ldw, N, K, ldw, bm);
        if (rc) return rc;
        rc = gm_make_map(&map_x, x, M, K, ldx, p.NB);
        if (rc) return rc;
    }
    const int smem = 1024 + n_stages * stage_bytes + tail;
    const int grid = p.n_units < n_sm ? p.n_units : n_sm;
    auto launch = [&](auto kernel) -> int {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return 1000 + (int)e;
        IL_LAUNCH(kernel, grid, GM_THREADS, smem, stream, map_w, map_w2, map_x, p);
        return IL_OK;
    };
    if (bm == 64) {
        if (glu) rc = kblk == 4 ? launch(gemm_mid_kernel<4, 2, 64>) : kblk == 2 ? launch(gemm_mid_kernel<2, 2, 64>) : launch(gemm_mid_kernel<1, 2, 64>);
        else rc = kblk == 4 ? launch(gemm_mid_kernel<4, 1, 64>) : launch(gemm_mid_kernel<2, 1, 64>);
    } else {
        if (glu) rc = kblk == 4 ? launch(gemm_mid_kernel<4, 2, 128>) : kblk == 2 ? launch(gemm_mid_kernel<2, 2, 128>) : launch(gemm_mid_kernel<1, 2, 128>);
        else rc = kblk == 4 ? launch(gemm_mid_kernel<4, 1, 128>) : launch(gemm_mid_kernel<2, 1, 128>);
    }
    if (rc) return rc;
    IL_LAUNCH_CHECK();
    return IL_OK;
}
