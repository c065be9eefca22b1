// SwiGLU on a fused gate-up activation: out[t,i] = silu(gu[t,i]) * gu[t,I+i], computed in f32.
// Also a bias add for library matrix products that have no bias epilogue.
#include "common.cuh"

template <typename TA>
__global__ void swiglu_kernel(const TA* __restrict__ gu, TA* __restrict__ out, int I, size_t total) {
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; idx < total; idx += stride) {
        const size_t t = idx / I;
        const int i = (int)(idx - t * I);
        const float g = il_to_f(gu[t * 2 * I + i]);
        const float u = il_to_f(gu[t * 2 * I + I + i]);
        out[idx] = il_from_f<TA>(sizeof(TA) == 2 ? il_silu_mul_fast(g, u) : g / (1.f + expf(-g)) * u);
    }
}

// 8 bfloat16 (or 4 float) per thread and access; I must be a multiple of the vector width.
template <typename TA, int VEC>
__global__ void swiglu_vec_kernel(const TA* __restrict__ gu, TA* __restrict__ out, int I, size_t total_vec) {
    const int ivec = I / VEC;
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; idx < total_vec; idx += stride) {
        const size_t t = idx / ivec;
        const int i = (int)(idx - t * ivec) * VEC;
        const uint4 gq = *reinterpret_cast<const uint4*>(gu + t * 2 * I + i);
        const uint4 uq = *reinterpret_cast<const uint4*>(gu + t * 2 * I + I + i);
        uint4 oq;
        const TA* gp = reinterpret_cast<const TA*>(&gq);
        const TA* up = reinterpret_cast<const TA*>(&uq);
        TA* op = reinterpret_cast<TA*>(&oq);
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
            const float g = il_to_f(gp[k]), u = il_to_f(up[k]);
            op[k] = il_from_f<TA>(sizeof(TA) == 2 ? il_silu_mul_fast(g, u) : g / (1.f + expf(-g)) * u);
        }
        *reinterpret_cast<uint4*>(out + t * I + i) = oq;
    }
}

template <typename TA>
__global__ void add_bias_kernel(TA* __restrict__ y, const void* __restrict__ b, int b_kind, int N, size_t total) {
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; idx < total; idx += stride) {
        const int n = (int)(idx % N);
        y[idx] = il_from_f<TA>(il_to_f(y[idx]) + il_load_any(b, b_kind, n));
    }
}

static inline int grid_for(size_t total, int threads) {
    size_t g = (total + threads - 1) / threads;
    const size_t cap = 148 * 16;
    return (int)(g > cap ? cap : g);
}

IL_EXPORT int il_swiglu(const void* gu, void* out, int act_kind, int T, int I, cudaStream_t stream) {
    if (T <= 0) return IL_OK;
    if (I <= 0) return IL_BAD_ARG;
    const size_t total = (size_t)T * I;
    if (act_kind == IL_BF16 && I % 8 == 0) {
        const size_t tv = total / 8;
        size_t g = (tv + 255) / 256;
        if (g > 148 * 32) g = 148 * 32;
        swiglu_vec_kernel<__nv_bfloat16, 8><<<(int)g, 256, 0, stream>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, I, tv);
        IL_LAUNCH_CHECK();
        return IL_OK;
    }
    if (act_kind == IL_F32 && I % 4 == 0) {
        const size_t tv = total / 4;
        size_t g = (tv + 255) / 256;
        if (g > 148 * 32) g = 148 * 32;
        swiglu_vec_kernel<float, 4><<<(int)g, 256, 0, stream>>>((const float*)gu, (float*)out, I, tv);
        IL_LAUNCH_CHECK();
        return IL_OK;
    }
    const int threads = 256, grid = grid_for(total, threads);
    if (act_kind == IL_F32)
        swiglu_kernel<float><<<grid, threads, 0, stream>>>((const float*)gu, (float*)out, I, total);
    else if (act_kind == IL_BF16)
        swiglu_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, I, total);
    else
        return IL_BAD_ARG;
    IL_LAUNCH_CHECK();
    return IL_OK;
}

IL_EXPORT int il_add_bias(void* y, int act_kind, const void* bias, int bias_kind, int T, int N, cudaStream_t stream) {
    if (T <= 0) return IL_OK;
    if (N <= 0) return IL_BAD_ARG;
    const size_t total = (size_t)T * N;
    const int threads = 256, grid = grid_for(total, threads);
    if (act_kind == IL_F32)
        add_bias_kernel<float><<<grid, threads, 0, stream>>>((float*)y, bias, bias_kind, N, total);
    else if (act_kind == IL_BF16)
        add_bias_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>((__nv_bfloat16*)y, bias, bias_kind, N, total);
    else
        return IL_BAD_ARG;
    IL_LAUNCH_CHECK();
    return IL_OK;
}
