// True 32-bit matrix product on the FP32 pipes (FFMA only; no tensor-core or TF32 mode):
//   C[M,N] = alpha * A[M,K] * W[N,K]^T (+ bias[N])
// A and W are row-major with K contiguous (the layout of activations and of checkpoint weights).
// Every output element is one accumulator that adds its K products in index order, in every
// tile shape, so a row's result is bit-identical whatever else is in the batch.
#include "common.cuh"

template <int BM, int BN, int TM, int TN>
__global__ void __launch_bounds__(256) gemm_f32_kernel(const float* __restrict__ A, int lda, const float* __restrict__ W, int ldw,
                                                       float* __restrict__ C, int ldc, const float* __restrict__ bias, float alpha,
                                                       int M, int N, int K) {
    constexpr int BK = 16;
    static_assert((BM / TM) * (BN / TN) == 256, "256 threads");
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid % (BN / TN), ty = tid / (BN / TN);
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int idx = tid; idx < BM * BK; idx += 256) {
            const int r = idx / BK, k = idx - r * BK;
            const int gm = m0 + r, gk = k0 + k;
            As[k][r] = (gm < M && gk < K) ? A[(size_t)gm * lda + gk] : 0.f;
        }
        for (int idx = tid; idx < BN * BK; idx += 256) {
            const int r = idx / BK, k = idx - r * BK;
            const int gn = n0 + r, gk = k0 + k;
            Ws[k][r] = (gn < N && gk < K) ? W[(size_t)gn * ldw + gk] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = Ws[k][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int gm = m0 + ty * TM + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int gn = n0 + tx * TN + j;
            if (gn >= N) continue;
            float v = alpha * acc[i][j];
            if (bias) v += bias[gn];
            C[(size_t)gm * ldc + gn] = v;
        }
    }
}

IL_EXPORT int il_gemm_f32(const float* A, int lda, const float* W, int ldw, float* C, int ldc, const float* bias,
                          float alpha, int M, int N, int K, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return IL_OK;
    if (K <= 0 || lda < K || ldw < K || ldc < N) return IL_BAD_ARG;
    if (M <= 16) {
        dim3 grid((N + 255) / 256, (M + 15) / 16);
        gemm_f32_kernel<16, 256, 1, 16><<<grid, 256, 0, stream>>>(A, lda, W, ldw, C, ldc, bias, alpha, M, N, K);
    } else if (M <= 64) {
        dim3 grid((N + 63) / 64, (M + 63) / 64);
        gemm_f32_kernel<64, 64, 4, 4><<<grid, 256, 0, stream>>>(A, lda, W, ldw, C, ldc, bias, alpha, M, N, K);
    } else {
        dim3 grid((N + 127) / 128, (M + 127) / 128);
        gemm_f32_kernel<128, 128, 8, 8><<<grid, 256, 0, stream>>>(A, lda, W, ldw, C, ldc, bias, alpha, M, N, K);
    }
    IL_LAUNCH_CHECK();
    return IL_OK;
}
