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

// ---- a residual add and an RMSNorm between two of these products, without a kernel of its own ------------------------
// The product before (o or down projection, gemm_skinny_resid_kernel) adds its result into the float32 residual, writes
// xw = residual * norm weight as bfloat16 and, per block of 16 columns and row, the sum of the residual's squares. The
// product after (gate+up or q/k/v) reads xw as its activations and these sums, and multiplies its results by
// rstd = rsqrt(sum / H + eps): (h * w * rstd) . W = rstd * ((h * w) . W). Sums are added in a fixed order.
struct GsNormIn {
    const float* partial;                         // [M][n_partial] sums of squares, or null: the activations are normalised already
    int n_partial;                                // <= 256
    float inv_h, eps;
};
constexpr int GS_NORM_MAX_PARTIALS = 256;

// Warp w fetches the partial sums of rows w (and w + 8); called right after the wait, summed up after the main loop.
template <int NT>
__device__ __forceinline__ void gs_norm_fetch(float (&pv)[NT][8], const GsNormIn& ni, int M, int warp, int lane) {
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        const int m = t * 8 + warp;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int k = lane + 32 * i;
            pv[t][i] = (ni.partial && m < M && k < ni.n_partial) ? ni.partial[(size_t)m * ni.n_partial + k] : 0.f;
        }
    }
}
template <int NT>
__device__ __forceinline__ void gs_norm_finish(float* rstd_s, const float (&pv)[NT][8], const GsNormIn& ni, int warp, int lane) {
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        float s = ((pv[t][0] + pv[t][1]) + (pv[t][2] + pv[t][3])) + ((pv[t][4] + pv[t][5]) + (pv[t][6] + pv[t][7]));
        s = il_warp_sum(s);
        if (lane == 0) rstd_s[t * 8 + warp] = ni.partial ? rsqrtf(s * ni.inv_h + ni.eps) : 1.f;
    }
}

// NT: 8-row groups of x (1: M <= 8, 2: M <= 16). GLU: 0 plain, 1 SwiGLU (W holds N gate rows, then N up rows). U: blocks in flight.
template <int NT, int GLU, int U, typename TO>
__global__ void __launch_bounds__(GS_WARPS * 32, 2) gemm_skinny_kernel(const __nv_bfloat16* __restrict__ x, int ldx,
                                                                    const __nv_bfloat16* __restrict__ W, int ldw, TO* __restrict__ out,
                                                                    int ldo, const float* __restrict__ bias, float alpha, int M, int N, int K,
                                                                    const GsNormIn ni) {
    constexpr int NW = 1;
    constexpr int ROWS = GLU ? 8 : 16;            // outputs per activation row and tile: 16 rows, or 8 gate rows with their 8 up rows
    __shared__ float part[GS_WARPS][NW][NT][16][8];
    __shared__ float rstd_s[NT * 8];
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
    float pv[NT][8];
    if (GLU) gs_norm_fetch<NT>(pv, ni, M, warp, lane);
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
    if (GLU) gs_norm_finish<NT>(rstd_s, pv, ni, warp, lane);
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
        const float an = GLU ? __fmul_rn(alpha, rstd_s[m]) : alpha;     // the norm's 1/rms, where the activations came without it
        float y = __fmaf_rn(an, s0, bias ? bias[n] : 0.f);      // spelled out as one fused multiply-add: the same bits from every build of this line
        if (GLU) {
            const float u = __fmaf_rn(an, s1, bias ? bias[N + n] : 0.f);
            y = il_silu_mul_fast(y, u);
        }
        gs_store<TO>(out + (size_t)m * ldo + n, y);
    }
}

template <int NT, int GLU, typename TO>
static cudaError_t gs_launch(const void* x, int ldx, const void* W, int ldw, void* out, int ldo, const float* bias, float alpha, int M, int N,
                      int K, cudaStream_t stream, const GsNormIn& ni = GsNormIn{nullptr, 0, 0.f, 0.f}) {
    constexpr int U = NT == 1 ? 8 : 4;
    constexpr int ROWS = GLU ? 8 : 16;
    return il_launch(gemm_skinny_kernel<NT, GLU, U, TO>, dim3((N + ROWS - 1) / ROWS), dim3(GS_WARPS * 32), 0, stream,
              (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)W, ldw, (TO*)out, ldo, bias, alpha, M, N, K, ni);
}

// glu = 1: W is [2N, K] (N gate rows, then N up rows), bias [2N], out[M,N] = silu(alpha*x.Wg^T + bg) * (alpha*x.Wu^T + bu).
// norm_partial (glu only, may be null): x is residual * norm weight and still wants its 1/rms, from these sums of squares
// [M][n_partial] (n_partial <= 256, H = the width they were summed over).
IL_EXPORT int il_gemm_skinny(const void* x, int ldx, const void* W, int ldw, void* out, int out_kind, int ldo, const float* bias,
                             float alpha, int M, int N, int K, int glu, const float* norm_partial, int n_partial, int norm_h,
                             float norm_eps, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return IL_OK;
    if (norm_partial && (!glu || n_partial <= 0 || n_partial > GS_NORM_MAX_PARTIALS || norm_h <= 0)) return IL_UNSUPPORTED;
    const GsNormIn ni{norm_partial, n_partial, norm_partial ? 1.f / (float)norm_h : 0.f, norm_eps};
    if (M > 16 || K <= 0 || (K & 7) || (ldx & 7) || (ldw & 7) || ldx < K || ldw < K || ldo < N) return IL_UNSUPPORTED;
    if (out_kind != IL_F32 && out_kind != IL_BF16) return IL_BAD_ARG;
    if (glu && out_kind != IL_BF16) return IL_UNSUPPORTED;
    cudaError_t e;
    if (M <= 8) {
        if (glu) e = gs_launch<1, 1, __nv_bfloat16>(x, ldx, W, ldw, out, ldo, bias, alpha, M, N, K, stream, ni);
        else if (out_kind == IL_BF16) e = gs_launch<1, 0, __nv_bfloat16>(x, ldx, W, ldw, out, ldo, bias, alpha, M, N, K, stream);
        else e = gs_launch<1, 0, float>(x, ldx, W, ldw, out, ldo, bias, alpha, M, N, K, stream);
    } else {
        if (glu) e = gs_launch<2, 1, __nv_bfloat16>(x, ldx, W, ldw, out, ldo, bias, alpha, M, N, K, stream, ni);
        else if (out_kind == IL_BF16) e = gs_launch<2, 0, __nv_bfloat16>(x, ldx, W, ldw, out, ldo, bias, alpha, M, N, K, stream);
        else e = gs_launch<2, 0, float>(x, ldx, W, ldw, out, ldo, bias, alpha, M, N, K, stream);
    }
    if (e != cudaSuccess) return 1000 + (int)e;
    IL_LAUNCH_CHECK();
    return IL_OK;
}

// ---- the q/k/v projection of a decode step with the rotary encoding and the cache write in its epilogue -------------
// out[M, (nh + 2 nkv) hd] = x . W^T (+ bias) as above, then q and k heads rotated (rotate-half pairs (d, d + rot/2),
// angle pos * inv_freq[d], cos and sin times mscale) and k, v written to their token's slot of the paged cache: what
// rope_store does as a kernel of its own. A block's 16 rows of W are, for the rotated part of a head, 8 rows at
// d0.. and the 8 rows at d0 + rot/2.. they pair with (the SwiGLU tiling in another guise); elsewhere 16 rows in a row.
// The product is rounded to bfloat16 before it is rotated, as it is when the two kernels run one after the other, so a
// token's keys do not depend on which path it took. rot and head_dim - rot must be multiples of 16.
struct GsRope {
    const int* tok_pos;
    const int* tok_entry;
    const int* block_table;
    int bt_stride;
    __nv_bfloat16* cache;                         // [page][2][nkv][page_size][hd], or null: nothing is stored
    int page_size, nh, nkv, hd, rot;
    const float* inv_freq;
    float mscale;
};

template <int NT, int U>
__global__ void __launch_bounds__(GS_WARPS * 32, 2) gemm_skinny_rope_kernel(const __nv_bfloat16* x, int ldx,
                                                                         const __nv_bfloat16* __restrict__ W, int ldw,
                                                                         __nv_bfloat16* __restrict__ out, int ldo,
                                                                         const float* __restrict__ bias, float alpha, int M, int K,
                                                                         const GsRope rp, const GsNormIn ni) {
    __shared__ float part[GS_WARPS][NT][16][8];
    __shared__ float rstd_s[NT * 8];
    __shared__ float cs[NT * 8][8], sn[NT * 8][8];
    __shared__ long long slot[NT * 8];            // element offset of the token's K slot of kv head 0 in the cache, or -1
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = lane >> 2, c = lane & 3;
    const int tiles_per_head = rp.hd >> 4, half = rp.rot >> 1;
    const int j = blockIdx.x / tiles_per_head, tl = blockIdx.x - j * tiles_per_head;    // head (q, then k, then v) and tile in it
    const bool rotated = j < rp.nh + rp.nkv && tl < (rp.rot >> 4);
    const int d0 = rotated ? tl * 8 : (j < rp.nh + rp.nkv ? rp.rot + (tl - (rp.rot >> 4)) * 16 : tl * 16);
    const int step = rotated ? half : 8;          // distance between the two rows a lane reads, = between a tile's two halves
    const int n_lo = j * rp.hd + d0;              // output column of the tile's row 0; row 8 + i is column n_lo + step + i
    const __nv_bfloat16* wrow[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) wrow[h] = W + (size_t)(n_lo + r + h * step) * ldw;
    // positions, slots and angles come with the step's descriptors: made ready while the kernel before still runs
    for (int i = threadIdx.x; i < NT * 8 * 8; i += GS_WARPS * 32) {
        const int m = i >> 3, nl = i & 7;
        float sv = 0.f, cv = 1.f;
        if (rotated && m < M) {
            sincosf((float)rp.tok_pos[m] * rp.inv_freq[d0 + nl], &sv, &cv);
            sv *= rp.mscale;
            cv *= rp.mscale;
        }
        sn[m][nl] = sv;
        cs[m][nl] = cv;
    }
    if (threadIdx.x < NT * 8) {
        const int m = threadIdx.x;
        long long off = -1;
        if (m < M && rp.cache && j >= rp.nh) {
            const int pos = rp.tok_pos[m];
            const int page = rp.block_table[(size_t)rp.tok_entry[m] * rp.bt_stride + pos / rp.page_size];
            if (page >= 0) off = ((long long)page * 2 * rp.nkv * rp.page_size + pos % rp.page_size) * rp.hd;
        }
        slot[m] = off;
    }
    il_pdl_begin();
    float pv[NT][8];
    gs_norm_fetch<NT>(pv, ni, M, warp, lane);
    const __nv_bfloat16* xrow[NT];
#pragma unroll
    for (int t = 0; t < NT; ++t) xrow[t] = (t * 8 + r < M) ? x + (size_t)(t * 8 + r) * ldx : nullptr;
    float acc[NT][4];
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[t][q] = 0.f;
    const int nkb = (K + 31) >> 5;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    for (int kb0 = warp; kb0 < nkb; kb0 += GS_WARPS * U) {
        uint4 a[U][2], b[U][NT];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int k = (kb0 + u * GS_WARPS) * 32 + c * 8;
            const bool ok = k < K;
            a[u][0] = ok ? gs_ld_stream(wrow[0] + k) : zero;
            a[u][1] = ok ? gs_ld_stream(wrow[1] + k) : zero;
#pragma unroll
            for (int t = 0; t < NT; ++t) b[u][t] = (ok && xrow[t]) ? gs_ld(xrow[t] + k) : zero;
        }
        __syncwarp();                             // keeps every load above issued before the first product waits for one
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                gs_mma(acc[t], a[u][0].x, a[u][1].x, a[u][0].y, a[u][1].y, b[u][t].x, b[u][t].y);
                gs_mma(acc[t], a[u][0].z, a[u][1].z, a[u][0].w, a[u][1].w, b[u][t].z, b[u][t].w);
            }
    }
    il_pdl_tail();
    gs_norm_finish<NT>(rstd_s, pv, ni, warp, lane);
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        part[warp][t][r][c * 2] = acc[t][0];
        part[warp][t][r][c * 2 + 1] = acc[t][1];
        part[warp][t][r + 8][c * 2] = acc[t][2];
        part[warp][t][r + 8][c * 2 + 1] = acc[t][3];
    }
    __syncthreads();
    const bool to_cache = j >= rp.nh;
    const int kv = j >= rp.nh + rp.nkv ? 1 : 0, g = j - rp.nh - kv * rp.nkv;            // for k and v heads
    const size_t head_off = ((size_t)kv * rp.nkv + (to_cache ? g : 0)) * rp.page_size * rp.hd;
    for (int idx = threadIdx.x; idx < NT * 8 * 8; idx += GS_WARPS * 32) {
        const int nl = idx & 7, m = idx >> 3;     // consecutive threads: consecutive output columns
        if (m >= M) continue;
        const int t = m >> 3, mc = m & 7;
        float s0 = 0.f, s1 = 0.f;
#pragma unroll
        for (int w = 0; w < GS_WARPS; ++w) {
            s0 += part[w][t][nl][mc];
            s1 += part[w][t][nl + 8][mc];
        }
        const int n1 = n_lo + nl, n2 = n1 + step;
        // rounded as the product alone would store them, then rotated
        const float an = alpha * rstd_s[m];       // the norm's 1/rms, where the activations came without it (else 1)
        const float y1 = __bfloat162float(__float2bfloat16_rn(an * s0 + (bias ? bias[n1] : 0.f)));
        const float y2 = __bfloat162float(__float2bfloat16_rn(an * s1 + (bias ? bias[n2] : 0.f)));
        const float cv = cs[m][nl], sv = sn[m][nl];
        const __nv_bfloat16 lo = __float2bfloat16_rn(rotated ? y1 * cv - y2 * sv : y1);
        const __nv_bfloat16 hi = __float2bfloat16_rn(rotated ? y2 * cv + y1 * sv : y2);
        out[(size_t)m * ldo + n1] = lo;
        out[(size_t)m * ldo + n2] = hi;
        if (to_cache && slot[m] >= 0) {
            __nv_bfloat16* dst = rp.cache + (size_t)slot[m] + head_off + (d0 + nl);
            dst[0] = lo;
            dst[step] = hi;
        }
    }
}

// The fused form for 1..16 rows; the shapes it takes: rot and head_dim - rot multiples of 16 (rot may be 0).
IL_EXPORT int il_gemm_skinny_rope(const void* x, int ldx, const void* W, int ldw, void* out, int ldo, const float* bias, float alpha,
                                  int M, int K, const int* tok_pos, const int* tok_entry, const int* block_table, int bt_stride,
                                  void* cache, int page_size, int nh, int nkv, int hd, int rot, const float* inv_freq, float mscale,
                                  const float* norm_partial, int n_partial, int norm_h, float norm_eps, cudaStream_t stream) {
    if (M <= 0) return IL_OK;
    if (norm_partial && (n_partial <= 0 || n_partial > GS_NORM_MAX_PARTIALS || norm_h <= 0)) return IL_UNSUPPORTED;
    const GsNormIn ni{norm_partial, n_partial, norm_partial ? 1.f / (float)norm_h : 0.f, norm_eps};
    const int N = (nh + 2 * nkv) * hd;
    if (M > 16 || K <= 0 || (K & 7) || (ldx & 7) || (ldw & 7) || ldx < K || ldw < K || ldo < N) return IL_UNSUPPORTED;
    if (nh <= 0 || nkv <= 0 || hd <= 0 || (hd & 15) || rot < 0 || rot > hd || (rot & 15) || page_size <= 0) return IL_UNSUPPORTED;
    if (rot > 0 && !inv_freq) return IL_BAD_ARG;
    GsRope rp{tok_pos, tok_entry, block_table, bt_stride, (__nv_bfloat16*)cache, page_size, nh, nkv, hd, rot, inv_freq, mscale};
    cudaError_t e;
    if (M <= 8)
        e = il_launch(gemm_skinny_rope_kernel<1, 8>, dim3(N / 16), dim3(GS_WARPS * 32), 0, stream, (const __nv_bfloat16*)x, ldx,
                      (const __nv_bfloat16*)W, ldw, (__nv_bfloat16*)out, ldo, bias, alpha, M, K, rp, ni);
    else
        e = il_launch(gemm_skinny_rope_kernel<2, 4>, dim3(N / 16), dim3(GS_WARPS * 32), 0, stream, (const __nv_bfloat16*)x, ldx,
                      (const __nv_bfloat16*)W, ldw, (__nv_bfloat16*)out, ldo, bias, alpha, M, K, rp, ni);
    if (e != cudaSuccess) return 1000 + (int)e;
    IL_LAUNCH_CHECK();
    return IL_OK;
}


// ---- the o or down projection with the residual add and the next norm's inputs in its epilogue ----------------------
// y = alpha * x . W^T (+ bias), rounded to bfloat16 as the product alone would store it; resid += bscale * y (float32, in
// place); xw = resid * norm_w as bfloat16; sumsq[m][block] = sum of resid^2 over the block's 16 columns. N = the width of
// the residual stream. What add_rmsnorm does, but for the division by the rms, which the next product applies.
template <int NT, int U>
__global__ void __launch_bounds__(GS_WARPS * 32, 2) gemm_skinny_resid_kernel(const __nv_bfloat16* __restrict__ x, int ldx,
                                                                          const __nv_bfloat16* __restrict__ W, int ldw,
                                                                          const float* __restrict__ bias, float alpha, int M, int N, int K,
                                                                          float* resid, float bscale, const void* __restrict__ norm_w,
                                                                          int norm_w_kind, __nv_bfloat16* __restrict__ xw,
                                                                          float* __restrict__ sumsq) {
    __shared__ float part[GS_WARPS][NT][16][8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = lane >> 2, c = lane & 3;
    const int n0 = blockIdx.x * 16;
    const __nv_bfloat16* wrow[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        int n = n0 + r + 8 * h;
        if (n > N - 1) n = N - 1;                 // rows past the end are computed and dropped
        wrow[h] = W + (size_t)n * ldw;
    }
    il_pdl_begin();
    // What the epilogue adds to - the residual, the norm's weight, the bias of this thread's (row, column) - is asked for
    // now: read after the main loop it cost the kernel a round trip to memory at its very end.
    const int e_nl = threadIdx.x & 15, e_m = threadIdx.x >> 4, e_n = n0 + e_nl;
    const bool e_live = (int)threadIdx.x < NT * 8 * 16 && e_m < M && e_n < N;
    const float e_resid = e_live ? resid[(size_t)e_m * N + e_n] : 0.f;
    const float e_w = e_live ? il_load_any(norm_w, norm_w_kind, e_n) : 0.f;
    const float e_bias = (e_live && bias) ? bias[e_n] : 0.f;
    const __nv_bfloat16* xrow[NT];
#pragma unroll
    for (int t = 0; t < NT; ++t) xrow[t] = (t * 8 + r < M) ? x + (size_t)(t * 8 + r) * ldx : nullptr;
    float acc[NT][4];
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[t][q] = 0.f;
    const int nkb = (K + 31) >> 5;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    for (int kb0 = warp; kb0 < nkb; kb0 += GS_WARPS * U) {
        uint4 a[U][2], b[U][NT];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int k = (kb0 + u * GS_WARPS) * 32 + c * 8;
            const bool ok = k < K;
            a[u][0] = ok ? gs_ld_stream(wrow[0] + k) : zero;
            a[u][1] = ok ? gs_ld_stream(wrow[1] + k) : zero;
#pragma unroll
            for (int t = 0; t < NT; ++t) b[u][t] = (ok && xrow[t]) ? gs_ld(xrow[t] + k) : zero;
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                gs_mma(acc[t], a[u][0].x, a[u][1].x, a[u][0].y, a[u][1].y, b[u][t].x, b[u][t].y);
                gs_mma(acc[t], a[u][0].z, a[u][1].z, a[u][0].w, a[u][1].w, b[u][t].z, b[u][t].w);
            }
    }
    il_pdl_tail();
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        part[warp][t][r][c * 2] = acc[t][0];
        part[warp][t][r][c * 2 + 1] = acc[t][1];
        part[warp][t][r + 8][c * 2] = acc[t][2];
        part[warp][t][r + 8][c * 2 + 1] = acc[t][3];
    }
    __syncthreads();
    // one thread per (row, column): 16 consecutive lanes share a row and add up its squares by shuffles; warps beyond the
    // NT * 8 * 16 pairs have nothing to do and leave as a whole
    if ((int)threadIdx.x >= NT * 8 * 16) return;
    const int nl = e_nl, m = e_m;
    const int n = e_n;
    const int t = m >> 3, mc = m & 7;
    float h = 0.f;
    if (m < M && n < N) {
        float s0 = 0.f;
#pragma unroll
        for (int w = 0; w < GS_WARPS; ++w) s0 += part[w][t][nl][mc];
        const float y = __bfloat162float(__float2bfloat16_rn(alpha * s0 + e_bias));
        h = e_resid + bscale * y;
        resid[(size_t)m * N + n] = h;
        xw[(size_t)m * N + n] = __float2bfloat16_rn(h * e_w);
    }
    float sq = h * h;
    sq += __shfl_xor_sync(0xffffffffu, sq, 8);
    sq += __shfl_xor_sync(0xffffffffu, sq, 4);
    sq += __shfl_xor_sync(0xffffffffu, sq, 2);
    sq += __shfl_xor_sync(0xffffffffu, sq, 1);
    if (nl == 0 && m < M) sumsq[(size_t)m * gridDim.x + blockIdx.x] = sq;
}

// N = width of the residual stream; sumsq gets [M][ceil(N / 16)] floats (at most 256 a row: N <= 4096).
IL_EXPORT int il_gemm_skinny_resid(const void* x, int ldx, const void* W, int ldw, const float* bias, float alpha, int M, int N, int K,
                                   float* resid, float bscale, const void* norm_w, int norm_w_kind, void* xw, float* sumsq,
                                   cudaStream_t stream) {
    if (M <= 0 || N <= 0) return IL_OK;
    if (M > 16 || K <= 0 || (K & 7) || (ldx & 7) || (ldw & 7) || ldx < K || ldw < K) return IL_UNSUPPORTED;
    if ((N + 15) / 16 > GS_NORM_MAX_PARTIALS || !resid || !norm_w || !xw || !sumsq) return IL_UNSUPPORTED;
    if (norm_w_kind != IL_F32 && norm_w_kind != IL_BF16) return IL_BAD_ARG;
    cudaError_t e;
    if (M <= 8)
        e = il_launch(gemm_skinny_resid_kernel<1, 8>, dim3((N + 15) / 16), dim3(GS_WARPS * 32), 0, stream, (const __nv_bfloat16*)x, ldx,
                      (const __nv_bfloat16*)W, ldw, bias, alpha, M, N, K, resid, bscale, norm_w, norm_w_kind, (__nv_bfloat16*)xw, sumsq);
    else
        e = il_launch(gemm_skinny_resid_kernel<2, 4>, dim3((N + 15) / 16), dim3(GS_WARPS * 32), 0, stream, (const __nv_bfloat16*)x, ldx,
                      (const __nv_bfloat16*)W, ldw, bias, alpha, M, N, K, resid, bscale, norm_w, norm_w_kind, (__nv_bfloat16*)xw, sumsq);
    if (e != cudaSuccess) return 1000 + (int)e;
    IL_LAUNCH_CHECK();
    return IL_OK;
}
