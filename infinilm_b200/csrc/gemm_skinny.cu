// Matrix product for a few activation rows (decode): out[M,N] = alpha * x[M,K] . W[N,K]^T (+ bias), M <= 16.
// The weights are streamed once from HBM at full width; that is all this kernel is about.
//
//   A block owns 16 rows of W (for the SwiGLU form: 8 gate rows and the 8 up rows that go with
//   them, as the two halves of one tensor-core tile). Its 8 warps take the 32-wide K blocks in turn (warp w: blocks w, w+8, ...), so together
//   they read 512 contiguous bytes of each row per round. A lane loads 16 bytes of two W rows and
//   16 bytes of one x row per block; the tensor core (m16n8k16, f32 accumulation) sees W as the
//   A operand and x as B, both with the same permutation of K inside a block, which a dot product
//   does not notice. Several blocks of loads are issued before the first product. The warps' partial
//   sums are added in warp order in shared memory, so a row's result is the same bits whatever else
//   is in the batch, and the epilogue applies alpha, bias, and SiLU(gate)*up in f32.
//
// K must be a multiple of 8 (16-byte loads); rows of x and W must be 16-byte aligned.
#include "common.cuh"

constexpr int GS_WARPS = 8;

__device__ __forceinline__ uint4 gs_ld_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 gs_ld(const void* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ void gs_mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <typename TO> __device__ __forceinline__ void gs_store(TO* p, float v);
template <> __device__ __forceinline__ void gs_store<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void gs_store<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// NT: 8-row groups of x (1: M <= 8, 2: M <= 16). GLU: 0 plain, 1 SwiGLU (W holds N gate rows, then N up rows). U: blocks in flight.
template <int NT, int GLU, int U, typename TO>
__global__ void __launch_bounds__(GS_WARPS * 32) gemm_skinny_kernel(const __nv_bfloat16* __restrict__ x, int ldx,
                                                                    const __nv_bfloat16* __restrict__ W, int ldw, TO* __restrict__ out,
                                                                    int ldo, const float* __restrict__ bias, float alpha, int M, int N, int K) {
    constexpr int NW = 1;
    constexpr int ROWS = GLU ? 8 : 16;            // outputs per activation row and tile: 16 rows, or 8 gate rows with their 8 up rows
    __shared__ float part[GS_WARPS][NW][NT][16][8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = lane >> 2, c = lane & 3;
    const int n0 = blockIdx.x * ROWS;
    const __nv_bfloat16* wrow[NW][2];
#pragma unroll
    for (int s = 0; s < NW; ++s)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            int n = GLU ? n0 + r : n0 + r + 8 * h;
            if (n > N - 1) n = N - 1;             // rows past the end are computed and dropped
            wrow[s][h] = W + ((size_t)(GLU ? h : 0) * N + n) * ldw;
        }
    il_pdl_begin();
    const __nv_bfloat16* xrow[NT];
#pragma unroll
    for (int t = 0; t < NT; ++t) xrow[t] = (t * 8 + r < M) ? x + (size_t)(t * 8 + r) * ldx : nullptr;

    float acc[NW][NT][4];
#pragma unroll
    for (int s = 0; s < NW; ++s)
#pragma unroll
        for (int t = 0; t < NT; ++t)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[s][t][j] = 0.f;

    const int nkb = (K + 31) >> 5;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    for (int kb0 = warp; kb0 < nkb; kb0 += GS_WARPS * U) {
        uint4 a[U][NW][2], b[U][NT];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int k = (kb0 + u * GS_WARPS) * 32 + c * 8;
            const bool ok = k < K;
#pragma unroll
            for (int s = 0; s < NW; ++s) {
                a[u][s][0] = ok ? gs_ld_stream(wrow[s][0] + k) : zero;
                a[u][s][1] = ok ? gs_ld_stream(wrow[s][1] + k) : zero;
            }
#pragma unroll
            for (int t = 0; t < NT; ++t) b[u][t] = (ok && xrow[t]) ? gs_ld(xrow[t] + k) : zero;
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int s = 0; s < NW; ++s)
#pragma unroll
                for (int t = 0; t < NT; ++t) {
                    gs_mma(acc[s][t], a[u][s][0].x, a[u][s][1].x, a[u][s][0].y, a[u][s][1].y, b[u][t].x, b[u][t].y);
                    gs_mma(acc[s][t], a[u][s][0].z, a[u][s][1].z, a[u][s][0].w, a[u][s][1].w, b[u][t].z, b[u][t].w);
                }
    }
    il_pdl_tail();
#pragma unroll
    for (int s = 0; s < NW; ++s)
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            part[warp][s][t][r][c * 2] = acc[s][t][0];
            part[warp][s][t][r][c * 2 + 1] = acc[s][t][1];
            part[warp][s][t][r + 8][c * 2] = acc[s][t][2];
            part[warp][s][t][r + 8][c * 2 + 1] = acc[s][t][3];
        }
    __syncthreads();
    for (int idx = threadIdx.x; idx < NT * 8 * ROWS; idx += GS_WARPS * 32) {
        const int nl = idx % ROWS, m = idx / ROWS;   // consecutive threads: consecutive output columns
        const int n = n0 + nl;
        if (m >= M || n >= N) continue;
        const int t = m >> 3, mc = m & 7;
        float s0 = 0.f, s1 = 0.f;
#pragma unroll
        for (int w = 0; w < GS_WARPS; ++w) {
            s0 += part[w][0][t][nl][mc];
            if (GLU) s1 += part[w][0][t][nl + 8][mc];
        }
        float y = alpha * s0 + (bias ? bias[n] : 0.f);
        if (GLU) {
            const float u = alpha * s1 + (bias ? bias[N + n] : 0.f);
            y = y / (1.f + expf(-y)) * u;
        }
        gs_store<TO>(out + (size_t)m * ldo + n, y);
    }
}

template <int NT, int GLU, typename TO>
static cudaError_t gs_launch(const void* x, int ldx, const void* W, int ldw, void* out, int ldo, const float* bias, float alpha, int M, int N,
                      int K, cudaStream_t stream) {
    constexpr int U = NT == 1 ? 8 : 4;
    constexpr int ROWS = GLU ? 8 : 16;
    return il_launch(gemm_skinny_kernel<NT, GLU, U, TO>, dim3((N + ROWS - 1) / ROWS), dim3(GS_WARPS * 32), 0, stream,
              (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)W, ldw, (TO*)out, ldo, bias, alpha, M, N, K);
}

// glu = 1: W is [2N, K] (N gate rows, then N up rows), bias [2N], out[M,N] = silu(alpha*x.Wg^T + bg) * (alpha*x.Wu^T + bu).
IL_EXPORT int il_gemm_skinny(const void* x, int ldx, const void* W, int ldw, void* out, int out_kind, int ldo, const float* bias,
                             float alpha, int M, int N, int K, int glu, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return IL_OK;
    if (M > 16 || K <= 0 || (K & 7) || (ldx & 7) || (ldw & 7) || ldx < K || ldw < K || ldo < N) return IL_UNSUPPORTED;
    if (out_kind != IL_F32 && out_kind != IL_BF16) return IL_BAD_ARG;
    if (glu && out_kind != IL_BF16) return IL_UNSUPPORTED;
    cudaError_t e;
    if (M <= 8) {
        if (glu) e = gs_launch<1, 1, __nv_bfloat16>(x, ldx, W, ldw, out, ldo, bias, alpha, M, N, K, stream);
        else if (out_kind == IL_BF16) e = gs_launch<1, 0, __nv_bfloat16>(x, ldx, W, ldw, out, ldo, bias, alpha, M, N, K, stream);
        else e = gs_launch<1, 0, float>(x, ldx, W, ldw, out, ldo, bias, alpha, M, N, K, stream);
    } else {
        if (glu) e = gs_launch<2, 1, __nv_bfloat16>(x, ldx, W, ldw, out, ldo, bias, alpha, M, N, K, stream);
        else if (out_kind == IL_BF16) e = gs_launch<2, 0, __nv_bfloat16>(x, ldx, W, ldw, out, ldo, bias, alpha, M, N, K, stream);
        else e = gs_launch<2, 0, float>(x, ldx, W, ldw, out, ldo, bias, alpha, M, N, K, stream);
    }
    if (e != cudaSuccess) return 1000 + (int)e;
    IL_LAUNCH_CHECK();
    return IL_OK;
}
