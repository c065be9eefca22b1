// Residual add fused with RMSNorm.
//   x = resid[r] + branch_scale * branch[r]   (branch may be absent)
//   resid[r] = x                              (kept in f32; skipped when a row list is given)
//   out[i]  = x / sqrt(mean(x^2) + eps) * w
// Sum of squares, rsqrt and the scaling are f32; one block per row with a fixed thread count,
// so a row's result does not depend on what else is in the batch.
#include "common.cuh"

template <typename TA>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const TA* __restrict__ branch, float bscale,
                                   const void* __restrict__ w, int w_kind, float eps, TA* __restrict__ out,
                                   const int* __restrict__ rows, int H) {
    extern __shared__ float xs[];
    __shared__ float red[32];
    const int i = blockIdx.x;
    const int r = rows ? rows[i] : i;
    float* rr = resid + (size_t)r * H;
    const TA* br = branch ? branch + (size_t)r * H : nullptr;
    float ss = 0.f;
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        float x = rr[h];
        if (br) x += bscale * il_to_f(br[h]);
        xs[h] = x;
        ss += x * x;
        if (!rows && br) rr[h] = x;
    }
    ss = il_block_sum(ss, red);
    const float rstd = rsqrtf(ss / (float)H + eps);
    TA* o = out + (size_t)i * H;
    for (int h = threadIdx.x; h < H; h += blockDim.x)
        o[h] = il_from_f<TA>(xs[h] * rstd * il_load_any(w, w_kind, h));
}

// The same with 4 elements per thread and access: 16-byte loads of the residual, 8- or 16-byte loads of
// the branch and the weight, all of a thread's loads issued before the first use.
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ld4(const __nv_bfloat16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x), b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st4(__nv_bfloat16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&a);
    u.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = u;
}

template <typename TA, int MAXV>
__global__ void __launch_bounds__(256) add_rmsnorm_vec_kernel(float* resid, const TA* branch, float bscale,
                                                              const void* __restrict__ w, int w_kind, float eps, TA* __restrict__ out,
                                                              const int* __restrict__ rows, int H) {
    __shared__ float red[32];
    const int i = blockIdx.x;
    const int nv = H >> 2;                        // float4 groups in a row
    // the norm's weights and the row index do not come from the kernel before this one: read while it still runs
    float4 wv[MAXV];
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
        const int v = threadIdx.x + k * 256;
        wv[k] = v < nv ? (w_kind == IL_F32 ? ld4((const float*)w + 4 * v) : ld4((const __nv_bfloat16*)w + 4 * v)) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const int r = rows ? rows[i] : i;
    il_pdl_wait();
    float* rr = resid + (size_t)r * H;
    const TA* br = branch ? branch + (size_t)r * H : nullptr;
    float4 x[MAXV];
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
        const int v = threadIdx.x + k * 256;
        x[k] = v < nv ? ld4(rr + 4 * v) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (br) {
        float4 b[MAXV];
#pragma unroll
        for (int k = 0; k < MAXV; ++k) {
            const int v = threadIdx.x + k * 256;
            b[k] = v < nv ? ld4(br + 4 * v) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int k = 0; k < MAXV; ++k) {
            x[k].x += bscale * b[k].x;
            x[k].y += bscale * b[k].y;
            x[k].z += bscale * b[k].z;
            x[k].w += bscale * b[k].w;
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < MAXV; ++k) ss += x[k].x * x[k].x + x[k].y * x[k].y + x[k].z * x[k].z + x[k].w * x[k].w;
    if (!rows && br) {
#pragma unroll
        for (int k = 0; k < MAXV; ++k) {
            const int v = threadIdx.x + k * 256;
            if (v < nv) st4(rr + 4 * v, x[k]);
        }
    }
    ss = il_block_sum(ss, red);
    const float rstd = rsqrtf(ss / (float)H + eps);
    TA* o = out + (size_t)i * H;
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
        const int v = threadIdx.x + k * 256;
        if (v < nv) st4(o + 4 * v, make_float4(x[k].x * rstd * wv[k].x, x[k].y * rstd * wv[k].y, x[k].z * rstd * wv[k].z, x[k].w * rstd * wv[k].w));
    }
}

template <typename TA>
static int launch_vec(float* resid, const void* branch, float bscale, const void* w, int w_kind, float eps, void* out,
                      const int* rows, int n_rows, int H, cudaStream_t stream) {
    const int nv = H >> 2;
    if (nv <= 256 * 2)
        IL_LAUNCH((add_rmsnorm_vec_kernel<TA, 2>), n_rows, 256, 0, stream, resid, (const TA*)branch, bscale, w, w_kind, eps, (TA*)out, rows, H);
    else if (nv <= 256 * 4)
        IL_LAUNCH((add_rmsnorm_vec_kernel<TA, 4>), n_rows, 256, 0, stream, resid, (const TA*)branch, bscale, w, w_kind, eps, (TA*)out, rows, H);
    else
        IL_LAUNCH((add_rmsnorm_vec_kernel<TA, 8>), n_rows, 256, 0, stream, resid, (const TA*)branch, bscale, w, w_kind, eps, (TA*)out, rows, H);
    return 0;
}

IL_EXPORT int il_add_rmsnorm(float* resid, const void* branch, float bscale, const void* w, int w_kind,
                             float eps, void* out, int act_kind, const int* rows, int n_rows, int H,
                             cudaStream_t stream) {
    if (n_rows <= 0) return IL_OK;
    if (H <= 0) return IL_BAD_ARG;
    if (H % 4 == 0 && H <= 256 * 8 * 4 && (act_kind == IL_F32 || act_kind == IL_BF16)) {
        if (act_kind == IL_F32) launch_vec<float>(resid, branch, bscale, w, w_kind, eps, out, rows, n_rows, H, stream);
        else launch_vec<__nv_bfloat16>(resid, branch, bscale, w, w_kind, eps, out, rows, n_rows, H, stream);
        IL_LAUNCH_CHECK();
        return IL_OK;
    }
    const size_t smem = (size_t)H * sizeof(float);
    if (smem > 200 * 1024) return IL_UNSUPPORTED;
    const int threads = 256;
    if (act_kind == IL_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(add_rmsnorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        add_rmsnorm_kernel<float><<<n_rows, threads, smem, stream>>>(resid, (const float*)branch, bscale, w, w_kind, eps, (float*)out, rows, H);
    } else if (act_kind == IL_BF16) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(add_rmsnorm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        add_rmsnorm_kernel<__nv_bfloat16><<<n_rows, threads, smem, stream>>>(resid, (const __nv_bfloat16*)branch, bscale, w, w_kind, eps, (__nv_bfloat16*)out, rows, H);
    } else
        return IL_BAD_ARG;
    IL_LAUNCH_CHECK();
    return IL_OK;
}
