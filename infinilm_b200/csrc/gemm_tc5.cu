// Matrix product on the 5th-generation tensor cores for a moderate number of activation rows
// (decode at large batch, short prompt portions): out[M,N] = alpha * x[M,K] . W[N,K]^T (+ bias), 16 < M <= 256.
//
//   The weights are the A operand: a tile is 128 rows of W, so the whole of W streams through the
//   tensor core once, and x (M rows, padded to a multiple of 16) is the B operand. The accumulator
//   D[128 x Mp] lives in tensor memory (TMEM), one W row per lane, one activation row per column.
//
//   Blocks are persistent (one per SM) and walk work units (tile, K slice). Roles by warp:
//     warp 0   producer: one lane issues TMA tensor copies (cp.async.bulk.tensor, 128-byte swizzle) of a
//              [128 x 64] box of W and a [Mp x 64] box of x into a ring of stages, completion on mbarriers;
//     warp 1   allocates TMEM; one lane issues tcgen05.mma (M 128, N Mp, K 16, bf16 -> f32) four times per
//              stage and commits: the commit frees the stage, and after a unit's last stage hands the
//              accumulator to the epilogue; two accumulators alternate so the next unit's products overlap it;
//     warps 2-5 epilogue: tcgen05.ld of their 32 lanes, alpha and bias in f32, stores of out (or of the f32
//              partials of a K slice, which il_tc5_finish adds up in slice order).
//   Rows of W past N, rows of x past M and columns past K are filled with zeros by the copy engine.
//
//   Every mbarrier wait is bounded; a wait that runs out sets *status, the roles leave their loops,
//   the block frees its TMEM and returns.
#include <cuda.h>

#include "common.cuh"

constexpr int TC_BM = 128;                        // W rows per tile (the MMA's M)
constexpr int TC_BK = 64;                         // K per stage: 128 bytes, the swizzle span
constexpr int TC_MAX_STAGES = 8;                  // the ring is as deep as shared memory allows, up to this
constexpr int TC_THREADS = 192;
constexpr unsigned TC_SPIN_LIMIT = 1u << 26;

__device__ __forceinline__ uint32_t tc_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void tc_mbar_init(uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void tc_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tc_mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool tc_mbar_wait(uint32_t bar, uint32_t parity) {
    for (unsigned spin = 0; spin < TC_SPIN_LIMIT; ++spin) {
        uint32_t done;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void tc_tma_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
// Shared-memory matrix descriptor, K-major, 128-byte swizzle: 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t tc_desc(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFF) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}\n"
                 ::"r"(d_tmem), "l"(a), "l"(b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                   "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
}

struct TcParams {
    int M, N, K, Mp;                              // Mp: M rounded up to a multiple of 16 (the MMA's N)
    int n_tiles, n_splits, chunks_per_split, n_chunks, n_stages;
    int ldo, out_kind;                            // direct output (n_splits == 1)
    float alpha;
    const float* bias;
    void* out;
    float* partial;                               // [n_splits][M][N] f32 when n_splits > 1
    int* status;
};

__global__ void __launch_bounds__(TC_THREADS, 1) gemm_tc5_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                 const __grid_constant__ CUtensorMap map_x, const TcParams p) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // stages must start on 1024-byte boundaries (the swizzle pattern repeats every 1024 bytes)
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int a_bytes = TC_BM * TC_BK * 2, b_bytes = p.Mp * TC_BK * 2;
    const int stage_bytes = a_bytes + ((b_bytes + 1023) & ~1023);
    const int TC_STAGES = p.n_stages;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + TC_STAGES * stage_bytes);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * TC_MAX_STAGES + 4);
    const uint32_t full0 = tc_smem(bars), empty0 = full0 + TC_MAX_STAGES * 8;
    const uint32_t tfull0 = empty0 + TC_MAX_STAGES * 8, tempty0 = tfull0 + 2 * 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // TMEM columns: two accumulators of Mp columns, a power of two >= 32
    uint32_t ncols = 32;
    while ((int)ncols < 2 * p.Mp) ncols <<= 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TC_STAGES; ++s) {
            tc_mbar_init(full0 + s * 8, 1);
            tc_mbar_init(empty0 + s * 8, 1);
        }
        for (int a = 0; a < 2; ++a) {
            tc_mbar_init(tfull0 + a * 8, 1);
            tc_mbar_init(tempty0 + a * 8, 4);     // one arrival per epilogue warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tc_smem(tmem_slot)), "r"(ncols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    const int n_units = p.n_tiles * p.n_splits;
    if (warp == 0) {
        // ---------------- producer ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
                const int tile = u / p.n_splits, split = u - tile * p.n_splits;
                const int c_lo = split * p.chunks_per_split, c_hi = min(p.n_chunks, c_lo + p.chunks_per_split);
                for (int c = c_lo; c < c_hi; ++c) {
                    if (!tc_mbar_wait(empty0 + stage * 8, phase ^ 1)) { atomicExch(p.status, 11); ok = false; break; }
                    const uint32_t full = full0 + stage * 8;
                    tc_mbar_expect_tx(full, (uint32_t)(a_bytes + b_bytes));
                    const uint32_t dst = tc_smem(smem + stage * stage_bytes);
                    tc_tma_2d(dst, &map_w, c * TC_BK, tile * TC_BM, full);
                    tc_tma_2d(dst + a_bytes, &map_x, c * TC_BK, 0, full);
                    if (++stage == TC_STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- tensor-core issue ----------------
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(p.Mp >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
            int stage = 0, acc = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
                const int tile = u / p.n_splits, split = u - tile * p.n_splits;
                const int c_lo = split * p.chunks_per_split, c_hi = min(p.n_chunks, c_lo + p.chunks_per_split);
                if (!tc_mbar_wait(tempty0 + acc * 8, acc_phase ^ 1)) { atomicExch(p.status, 12); break; }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * p.Mp);
                for (int c = c_lo; c < c_hi; ++c) {
                    if (!tc_mbar_wait(full0 + stage * 8, phase)) { atomicExch(p.status, 13); ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    const uint32_t sa = tc_smem(smem + stage * stage_bytes);
                    const uint64_t da = tc_desc(sa), db = tc_desc(sa + a_bytes);
#pragma unroll
                    for (int kk = 0; kk < TC_BK / 16; ++kk)   // 32 bytes further along K inside the swizzle span
                        tc_mma(d_tmem, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2), idesc, (c > c_lo || kk > 0) ? 1u : 0u);
                    tc_commit(empty0 + stage * 8);            // the stage is free once these products have read it
                    if (++stage == TC_STAGES) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                tc_commit(tfull0 + acc * 8);                  // the accumulator is complete
                if (++acc == 2) { acc = 0; acc_phase ^= 1; }
            }
        }
    } else {
        // ---------------- epilogue: warps 2..5 own TMEM lanes 32*(warp % 4) .. +31 ----------------
        const int q = warp & 3;
        int acc = 0;
        uint32_t acc_phase = 0;
        for (int u = blockIdx.x; u < n_units; u += gridDim.x) {
            const int tile = u / p.n_splits, split = u - tile * p.n_splits;
            if (!tc_mbar_wait(tfull0 + acc * 8, acc_phase)) { atomicExch(p.status, 14); break; }
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const int n = tile * TC_BM + q * 32 + lane;       // this lane's W row = output column
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * p.Mp);
            for (int j0 = 0; j0 < p.Mp; j0 += 16) {
                uint32_t v[16];
                tc_ld16(taddr + j0, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                if (n < p.N) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int m = j0 + j;
                        if (m >= p.M) break;
                        const float acc_v = __uint_as_float(v[j]);
                        if (p.n_splits > 1) {
                            p.partial[((size_t)split * p.M + m) * p.N + n] = acc_v;
                        } else {
                            const float y = p.alpha * acc_v + (p.bias ? p.bias[n] : 0.f);
                            if (p.out_kind == IL_F32) ((float*)p.out)[(size_t)m * p.ldo + n] = y;
                            else ((__nv_bfloat16*)p.out)[(size_t)m * p.ldo + n] = __float2bfloat16_rn(y);
                        }
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) tc_mbar_arrive(tempty0 + acc * 8);
            if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(ncols) : "memory");
    }
}

// out[m][n] = alpha * sum over slices of partial[s][m][n] (+ bias), slices added in order.
__global__ void tc5_finish_kernel(const float* __restrict__ partial, int n_splits, int M, int N, float alpha,
                                  const float* __restrict__ bias, void* __restrict__ out, int out_kind, int ldo) {
    const size_t total = (size_t)M * N;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int m = (int)(i / N), n = (int)(i - (size_t)m * N);
        float s = 0.f;
        for (int k = 0; k < n_splits; ++k) s += partial[(size_t)k * total + i];
        const float y = alpha * s + (bias ? bias[n] : 0.f);
        if (out_kind == IL_F32) ((float*)out)[(size_t)m * ldo + n] = y;
        else ((__nv_bfloat16*)out)[(size_t)m * ldo + n] = __float2bfloat16_rn(y);
    }
}

typedef CUresult (*tc_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static tc_encode_fn tc_encoder() {
    static tc_encode_fn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (tc_encode_fn)p;
    }
    return fn;
}

// A [rows x K] bfloat16 matrix with row stride ld, read in boxes of [box_rows x 64] with the 128-byte swizzle.
static int tc_make_map(CUtensorMap* map, const void* base, int rows, int K, int ld, int box_rows) {
    tc_encode_fn enc = tc_encoder();
    if (!enc) return IL_UNSUPPORTED;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)TC_BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 2000 + (int)r;
}

// How many K slices. In bytes moved at full bandwidth, a choice costs
//   rounds * (bytes of a unit) * SMs   (every round lasts as long as its slowest SM: one unit)
// + 2 * slices * M * N * 4             (the f32 partials are written and read once), for slices > 1;
// the cheapest wins, with at least 4 chunks of 64 per slice.
static int tc_pick_splits(int n_tiles, int n_chunks, int n_sm, int M, int N) {
    int best = 1;
    double best_cost = 0.0;
    for (int s = 1; s <= 16; s *= 2) {
        if (s > 1 && n_chunks / s < 4) break;
        const int cps = (n_chunks + s - 1) / s;
        const int units = n_tiles * ((n_chunks + cps - 1) / cps);
        const int rounds = (units + n_sm - 1) / n_sm;
        const double cost = (double)rounds * cps * (TC_BM * TC_BK * 2) * n_sm + (s > 1 ? 2.0 * s * M * (double)N * 4 : 0.0);
        if (s == 1 || cost < best_cost) { best_cost = cost; best = s; }
    }
    return best;
}

// Bytes of f32 scratch `partial` must hold for this shape (0: no K split is used).
IL_EXPORT long long il_gemm_tc5_scratch_bytes(int M, int N, int K) {
    int dev = 0, n_sm = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
    const int n_tiles = (N + TC_BM - 1) / TC_BM, n_chunks = (K + TC_BK - 1) / TC_BK;
    const int s = tc_pick_splits(n_tiles, n_chunks, n_sm, M, N);
    return s > 1 ? (long long)s * M * N * 4 : 0;
}

IL_EXPORT int il_gemm_tc5(const void* x, int ldx, const void* W, int ldw, void* out, int out_kind, int ldo, const float* bias,
                          float alpha, int M, int N, int K, float* partial, int* status, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return IL_OK;
    if (M > 256 || K <= 0 || (K & 7) || (ldx & 7) || (ldw & 7) || ldx < K || ldw < K || ldo < N || !status) return IL_UNSUPPORTED;
    if (((uintptr_t)x & 15) || ((uintptr_t)W & 15)) return IL_UNSUPPORTED;
    if (out_kind != IL_F32 && out_kind != IL_BF16) return IL_BAD_ARG;
    int dev = 0, n_sm = 148;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sm <= 0) n_sm = 148;

    TcParams p;
    p.M = M; p.N = N; p.K = K; p.Mp = (M + 15) & ~15;
    p.n_tiles = (N + TC_BM - 1) / TC_BM;
    p.n_chunks = (K + TC_BK - 1) / TC_BK;
    p.n_splits = tc_pick_splits(p.n_tiles, p.n_chunks, n_sm, M, N);
    p.chunks_per_split = (p.n_chunks + p.n_splits - 1) / p.n_splits;
    p.n_splits = (p.n_chunks + p.chunks_per_split - 1) / p.chunks_per_split;     // no empty slice
    if (p.n_splits > 1 && !partial) return IL_BAD_ARG;
    p.ldo = ldo; p.out_kind = out_kind; p.alpha = alpha; p.bias = bias; p.out = out; p.partial = partial; p.status = status;

    CUtensorMap map_w, map_x;
    int rc = tc_make_map(&map_w, W, N, K, ldw, TC_BM);
    if (rc) return rc;
    rc = tc_make_map(&map_x, x, M, K, ldx, p.Mp);
    if (rc) return rc;

    const int a_bytes = TC_BM * TC_BK * 2, b_bytes = p.Mp * TC_BK * 2;
    const int stage_bytes = a_bytes + ((b_bytes + 1023) & ~1023);
    const int tail = (2 * TC_MAX_STAGES + 4) * 8 + 16;
    int n_stages = (227 * 1024 - 1024 - tail) / stage_bytes;
    if (n_stages > TC_MAX_STAGES) n_stages = TC_MAX_STAGES;
    if (n_stages < 2) return IL_UNSUPPORTED;
    p.n_stages = n_stages;
    const int smem = 1024 + n_stages * stage_bytes + tail;
    static int attr_smem[64];
    if (dev >= 0 && dev < 64 && attr_smem[dev] < smem) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return 1000 + (int)e;
        attr_smem[dev] = smem;
    }
    const int n_units = p.n_tiles * p.n_splits;
    const int grid = n_units < n_sm ? n_units : n_sm;
    gemm_tc5_kernel<<<grid, TC_THREADS, smem, stream>>>(map_w, map_x, p);
    IL_LAUNCH_CHECK();
    if (p.n_splits > 1) {
        const size_t total = (size_t)M * N;
        int fg = (int)((total + 255) / 256);
        if (fg > n_sm * 8) fg = n_sm * 8;
        tc5_finish_kernel<<<fg, 256, 0, stream>>>(partial, p.n_splits, M, N, alpha, bias, out, out_kind, ldo);
        IL_LAUNCH_CHECK();
    }
    return IL_OK;
}
