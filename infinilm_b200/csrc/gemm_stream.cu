// Matrix product for a few activation rows (decode): out[M,N] = alpha * x[M,K] . W[N,K]^T (+ bias), M <= 16,
// built around the bulk asynchronous copy engine (TMA): the weights stream from HBM into a ring
// of shared-memory stages without passing through registers, so the bytes in flight do not
// depend on how the compiler schedules loads.
//
//   One persistent block per SM owns a contiguous range of weight rows (N / blocks of them, so every
//   block has the same work to within a row). It walks the range in tiles of 16 rows (SwiGLU form:
//   8 gate rows and the 8 up rows that go with them) and each tile in K chunks of 512.
//   Warp 8 is the producer: it waits for a free stage (mbarrier), lane 0 announces the bytes to come
//   and the lanes issue one bulk copy each, a row apiece: sixteen weight rows and the M rows of x
//   for the same K chunk (cp.async.bulk, completion counted on the stage's mbarrier).
//   Warps 0-7 are consumers: they wait for the stage, read their 16-byte pieces of two rows
//   (ld.shared.v4; rows are padded so that a quarter-warp hits distinct banks), the matching 16
//   bytes of x from the same stage, and feed the tensor core (m16n8k16, f32 accumulation; W is the A operand,
//   x the B operand, with the same permutation of K inside a 32-block on both sides). After a
//   chunk each consumer warp releases the stage. At the end of a tile the eight partial sums are
//   added in warp order in shared memory - a row's result is the same bits whatever else is in
//   the batch - and the epilogue applies alpha, bias and SiLU(gate)*up in f32.
//
//   Every mbarrier wait is bounded: after GS_SPIN_LIMIT polls the waiter sets *status and leaves
//   its loop; the host reads the status word. A stage's copies complete on their own.
//
// K must be a multiple of 8 (16-byte pieces); rows of x and W must be 16-byte aligned.
#include "common.cuh"

constexpr int GT_CONSUMERS = 8;
constexpr int GT_THREADS = (GT_CONSUMERS + 1) * 32;
constexpr int GT_KC = 512;                        // K elements per chunk
constexpr int GT_ROW_BYTES = GT_KC * 2 + 64;      // padded row of a stage
// A stage holds 16 weight rows and the 8*NT activation rows of the same K chunk.
template <int NT> struct GtCfg {
    static constexpr int STAGE_BYTES = (16 + 8 * NT) * GT_ROW_BYTES;
    static constexpr int STAGES = NT == 1 ? 6 : 5;
    static constexpr int PART_BYTES = 2 * GT_CONSUMERS * NT * 16 * 8 * 4;
    static constexpr int SMEM = STAGES * STAGE_BYTES + PART_BYTES + 2 * STAGES * 8;
};
constexpr unsigned GT_SPIN_LIMIT = 1u << 26;

__device__ __forceinline__ void gt_mbar_init(uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void gt_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void gt_mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
// Returns false if the phase did not complete within the poll limit.
__device__ __forceinline__ bool gt_mbar_wait(uint32_t bar, uint32_t parity) {
    for (unsigned spin = 0; spin < GT_SPIN_LIMIT; ++spin) {
        uint32_t done;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void gt_bulk_copy(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ uint4 gt_lds(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void gt_mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <typename TO> __device__ __forceinline__ void gt_store(TO* p, float v);
template <> __device__ __forceinline__ void gt_store<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void gt_store<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// NT: 8-row groups of x (1: M <= 8, 2: M <= 16). GLU: W holds N gate rows, then N up rows.
template <int NT, int GLU, typename TO>
__global__ void __launch_bounds__(GT_THREADS, 1) gemm_stream_kernel(const __nv_bfloat16* __restrict__ x, int ldx,
                                                                    const __nv_bfloat16* __restrict__ W, int ldw, TO* __restrict__ out,
                                                                    int ldo, const float* __restrict__ bias, float alpha, int M, int N, int K,
                                                                    int* __restrict__ status) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int ROWS = GLU ? 8 : 16;            // outputs per activation row and tile
    constexpr int GT_STAGES = GtCfg<NT>::STAGES, GT_STAGE_BYTES = GtCfg<NT>::STAGE_BYTES;
    float (*part)[GT_CONSUMERS][NT][16][8] =
        reinterpret_cast<float (*)[GT_CONSUMERS][NT][16][8]>(smem + GT_STAGES * GT_STAGE_BYTES);      // [2]
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + GT_STAGES * GT_STAGE_BYTES + GtCfg<NT>::PART_BYTES);
    const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(smem);
    const uint32_t full0 = (uint32_t)__cvta_generic_to_shared(bars), empty0 = full0 + GT_STAGES * 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < GT_STAGES; ++s) {
            gt_mbar_init(full0 + s * 8, 1);
            gt_mbar_init(empty0 + s * 8, GT_CONSUMERS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    __syncthreads();

    // This block's rows: [n_lo, n_hi) of the N output columns (gate rows for the SwiGLU form).
    const int n_lo = (int)(((long long)N * blockIdx.x) / gridDim.x), n_hi = (int)(((long long)N * (blockIdx.x + 1)) / gridDim.x);
    const int n_tiles = (n_hi - n_lo + ROWS - 1) / ROWS;
    const int n_chunks = (K + GT_KC - 1) / GT_KC;

    if (warp == GT_CONSUMERS) {
        // ---------------- producer ----------------
        // Lane l copies row l of the stage (SwiGLU form: lanes 0-7 the gate rows, 8-15 the up rows), so the
        // sixteen bulk copies of a stage are issued by one warp instruction.
        int stage = 0;
        uint32_t phase = 0;
        for (int t = 0; t < n_tiles; ++t) {
            const int row0 = n_lo + t * ROWS;
            const int rows_valid = min(ROWS, n_hi - row0);
            const int my = GLU ? (lane & 7) : lane;                       // row of the tile this lane copies
            const bool is_x = lane >= 16 && lane - 16 < M;                // lanes 16.. copy the activation rows of the chunk
            const bool active = (lane < 16 && my < rows_valid) || is_x;
            const __nv_bfloat16* src_row = is_x ? x + (size_t)(lane - 16) * ldx
                                                : W + (size_t)((GLU && lane >= 8 ? N : 0) + row0 + (active ? my : 0)) * ldw;
            for (int ch = 0; ch < n_chunks; ++ch) {
                const int k0 = ch * GT_KC;
                const uint32_t bytes = (uint32_t)(min(GT_KC, K - k0) * 2);
                if (!gt_mbar_wait(empty0 + stage * 8, phase ^ 1)) {
                    if (lane == 0) atomicExch(status, 1);
                    return;
                }
                const uint32_t full = full0 + stage * 8;
                if (lane == 0) gt_mbar_expect_tx(full, bytes * (rows_valid * (GLU ? 2 : 1) + M));
                __syncwarp();
                if (active) gt_bulk_copy(sbase + stage * GT_STAGE_BYTES + lane * GT_ROW_BYTES, src_row + k0, bytes, full);
                if (++stage == GT_STAGES) { stage = 0; phase ^= 1; }
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    const int r = lane >> 2, c = lane & 3;
    float acc[NT][4];
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[t][j] = 0.f;

    int stage = 0;
    uint32_t phase = 0;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    constexpr int BLOCKS_PER_WARP = GT_KC / 32 / GT_CONSUMERS;    // 32-wide K blocks of a chunk per consumer warp
    for (int t = 0; t < n_tiles; ++t) {
        for (int ch = 0; ch < n_chunks; ++ch) {
            const int k0 = ch * GT_KC;
            if (!gt_mbar_wait(full0 + stage * 8, phase)) {
                atomicExch(status, 2);
                return;
            }
            const uint32_t src = sbase + stage * GT_STAGE_BYTES + r * GT_ROW_BYTES + c * 16;
#pragma unroll
            for (int j = 0; j < BLOCKS_PER_WARP; ++j) {
                const int kl = (warp + j * GT_CONSUMERS) * 32;
                uint4 a0 = gt_lds(src + kl * 2), a1 = gt_lds(src + 8 * GT_ROW_BYTES + kl * 2);
                if (k0 + kl + c * 8 >= K) a0 = a1 = zero;           // past the end of K: the stage holds old bytes there
#pragma unroll
                for (int tt = 0; tt < NT; ++tt) {
                    // rows of x past M were never copied: their columns of the result are never stored
                    uint4 b = gt_lds(src + (16 + 8 * tt) * GT_ROW_BYTES + kl * 2);
                    if (k0 + kl + c * 8 >= K) b = zero;
                    gt_mma(acc[tt], a0.x, a1.x, a0.y, a1.y, b.x, b.y);
                    gt_mma(acc[tt], a0.z, a1.z, a0.w, a1.w, b.z, b.w);
                }
            }
            __syncwarp();
            if (lane == 0) gt_mbar_arrive(empty0 + stage * 8);
            if (++stage == GT_STAGES) { stage = 0; phase ^= 1; }
        }
        // end of a tile: add the warps' partial sums in warp order, write the outputs
        float (*p)[NT][16][8] = part[t & 1];
#pragma unroll
        for (int tt = 0; tt < NT; ++tt) {
            p[warp][tt][r][c * 2] = acc[tt][0];
            p[warp][tt][r][c * 2 + 1] = acc[tt][1];
            p[warp][tt][r + 8][c * 2] = acc[tt][2];
            p[warp][tt][r + 8][c * 2 + 1] = acc[tt][3];
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[tt][j] = 0.f;
        }
        asm volatile("bar.sync 1, %0;\n" ::"n"(GT_CONSUMERS * 32) : "memory");
        const int row0 = n_lo + t * ROWS;
        for (int idx = threadIdx.x; idx < NT * 8 * ROWS; idx += GT_CONSUMERS * 32) {
            const int nl = idx % ROWS, m = idx / ROWS;            // consecutive threads: consecutive output columns
            const int n = row0 + nl;
            if (m >= M || n >= n_hi) continue;
            const int tt = m >> 3, mc = m & 7;
            float s0 = 0.f, s1 = 0.f;
#pragma unroll
            for (int w = 0; w < GT_CONSUMERS; ++w) {
                s0 += p[w][tt][nl][mc];
                if (GLU) s1 += p[w][tt][nl + 8][mc];
            }
            float y = __fmaf_rn(alpha, s0, bias ? bias[n] : 0.f);      // spelled out: the same bits as gemm_skinny's epilogue
            if (GLU) {
                const float u = __fmaf_rn(alpha, s1, bias ? bias[N + n] : 0.f);
                y = il_silu_mul_fast(y, u);
            }
            gt_store<TO>(out + (size_t)m * ldo + n, y);
        }
    }
}

template <int NT, int GLU, typename TO>
static int gt_launch(const void* x, int ldx, const void* W, int ldw, void* out, int ldo, const float* bias, float alpha, int M, int N,
                     int K, int* status, cudaStream_t stream) {
    constexpr int SMEM = GtCfg<NT>::SMEM;
    static int n_sm[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return IL_BAD_ARG;
    if (!n_sm[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_stream_kernel<NT, GLU, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return 1000 + (int)e;
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
        n_sm[dev] = v;
    }
    constexpr int ROWS = GLU ? 8 : 16;
    const int max_blocks = (N + ROWS - 1) / ROWS;
    const int grid = n_sm[dev] < max_blocks ? n_sm[dev] : max_blocks;
    gemm_stream_kernel<NT, GLU, TO><<<grid, GT_THREADS, SMEM, stream>>>(
        (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)W, ldw, (TO*)out, ldo, bias, alpha, M, N, K, status);
    return 0;
}

// Same contract as il_gemm_skinny, plus `status`: a device int the kernel sets non-zero if a wait ran out.
IL_EXPORT int il_gemm_stream(const void* x, int ldx, const void* W, int ldw, void* out, int out_kind, int ldo, const float* bias,
                             float alpha, int M, int N, int K, int glu, int* status, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return IL_OK;
    if (M > 16 || K <= 0 || (K & 7) || (ldx & 7) || (ldw & 7) || ldx < K || ldw < K || ldo < N || !status) return IL_UNSUPPORTED;
    if (out_kind != IL_F32 && out_kind != IL_BF16) return IL_BAD_ARG;
    if (glu && out_kind != IL_BF16) return IL_UNSUPPORTED;
    int rc;
    if (M <= 8) {
        if (glu) rc = gt_launch<1, 1, __nv_bfloat16>(x, ldx, W, ldw, out, ldo, bias, alpha, M, N, K, status, stream);
        else if (out_kind == IL_BF16) rc = gt_launch<1, 0, __nv_bfloat16>(x, ldx, W, ldw, out, ldo, bias, alpha, M, N, K, status, stream);
        else rc = gt_launch<1, 0, float>(x, ldx, W, ldw, out, ldo, bias, alpha, M, N, K, status, stream);
    } else {
        if (glu) rc = gt_launch<2, 1, __nv_bfloat16>(x, ldx, W, ldw, out, ldo, bias, alpha, M, N, K, status, stream);
        else if (out_kind == IL_BF16) rc = gt_launch<2, 0, __nv_bfloat16>(x, ldx, W, ldw, out, ldo, bias, alpha, M, N, K, status, stream);
        else rc = gt_launch<2, 0, float>(x, ldx, W, ldw, out, ldo, bias, alpha, M, N, K, status, stream);
    }
    if (rc) return rc;
    IL_LAUNCH_CHECK();
    return IL_OK;
}
