// Shared helpers of the sm_100a kernels: element conversion, reductions, launch checks.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define IL_EXPORT extern "C" __attribute__((visibility("default")))

// Element kinds passed from the host as integers.
enum { IL_F32 = 0, IL_BF16 = 1 };

// Error codes returned by the entry points (0 = launched).
enum { IL_OK = 0, IL_BAD_ARG = -1, IL_UNSUPPORTED = -2 };

#define IL_LAUNCH_CHECK()                                         \
    do {                                                          \
        cudaError_t e__ = cudaGetLastError();                     \
        if (e__ != cudaSuccess) return 1000 + (int)e__;           \
    } while (0)

__device__ __forceinline__ float il_to_f(float x) { return x; }
__device__ __forceinline__ float il_to_f(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T il_from_f(float x);
template <> __device__ __forceinline__ float il_from_f<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 il_from_f<__nv_bfloat16>(float x) {
    return __float2bfloat16_rn(x);
}

// Reads element i of a vector stored as f32 or bf16.
__device__ __forceinline__ float il_load_any(const void* p, int kind, size_t i) {
    return kind == IL_F32 ? ((const float*)p)[i] : __bfloat162float(((const __nv_bfloat16*)p)[i]);
}

__device__ __forceinline__ float il_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float il_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result. `sh` holds 32 floats.
__device__ __forceinline__ float il_block_sum(float v, float* sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nw = (blockDim.x + 31) >> 5;
    v = il_warp_sum(v);
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    float t = (lane < nw) ? sh[lane] : 0.f;
    t = il_warp_sum(t);
    return t;
}
__device__ __forceinline__ float il_block_max(float v, float* sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nw = (blockDim.x + 31) >> 5;
    v = il_warp_max(v);
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    float t = (lane < nw) ? sh[lane] : -INFINITY;
    t = il_warp_max(t);
    return t;
}

// SiLU(g) * u for the bfloat16 path: exponential and division by the fast units (relative error near 2^-21, far below a
// bfloat16 step). The decode product's epilogue and the SwiGLU kernel both use it, so a token's activation does not
// depend on which of the two computed it. The float32 path keeps expf and a true division.
__device__ __forceinline__ float il_silu_mul_fast(float g, float u) { return __fmul_rn(__fdividef(g, __fadd_rn(1.f, __expf(-g))), u); }

// ---- programmatic dependent launch --------------------------------------------------------------
// Kernels of the decode path are launched so that the next kernel in the stream may become resident
// while this one drains (INFINILM_B200_PDL=0 turns it off). A kernel waits for its predecessor to have
// finished and flushed (il_pdl_begin) before it touches anything another kernel produces or reads, and
// lets its successor in once its main loop is over (il_pdl_tail; a kernel without one does so by ending).
// Both are no-ops in a kernel that was launched the ordinary way. A kernel may do, before its wait, whatever does not
// depend on its predecessor (read weights, step descriptors, cache pages of earlier tokens). What the predecessor
// writes must then NOT be read through a `const __restrict__` pointer: such loads count as read-only data for the
// whole kernel (ld.global.nc) and were seen scheduled above the wait, which replayed graphs then showed as wrong tokens. Measured on the 8B decode step at
// batch 8: 3.65 ms so, 3.70 ms without; with every kernel letting its successor in at its very start
// (IL_PDL_MODE 0) 6.7 ms, because waiting blocks of later kernels then crowd the SMs.
__device__ __forceinline__ void il_pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }
__device__ __forceinline__ void il_pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
// Where a kernel lets its successor in: IL_PDL_MODE 0 at its start, 1 after its main loop, 2 only by ending.
#ifndef IL_PDL_MODE
#define IL_PDL_MODE 1
#endif
__device__ __forceinline__ void il_pdl_begin() {
    if (IL_PDL_MODE == 0) il_pdl_launch_dependents();
    il_pdl_wait();
}
__device__ __forceinline__ void il_pdl_tail() {
    if (IL_PDL_MODE == 1) il_pdl_launch_dependents();
}

#include <cstdlib>
static inline bool il_pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("INFINILM_B200_PDL");
        on = (e && e[0] == '0') ? 0 : 1;
    }
    return on == 1;
}

template <typename... KArgs, typename... Args>
static inline cudaError_t il_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = il_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
#define IL_LAUNCH(kernel, grid, block, smem, stream, ...)                                                \
    do {                                                                                                   \
        cudaError_t e__ = il_launch(kernel, dim3(grid), dim3(block), (size_t)(smem), stream, __VA_ARGS__); \
        if (e__ != cudaSuccess) return 1000 + (int)e__;                                                   \
    } while (0)
