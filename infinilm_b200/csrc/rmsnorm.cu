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

IL_EXPORT int il_add_rmsnorm(float* resid, const void* branch, float bscale, const void* w, int w_kind,
                             float eps, void* out, int act_kind, const int* rows, int n_rows, int H,
                             cudaStream_t stream) {
    if (n_rows <= 0) return IL_OK;
    if (H <= 0) return IL_BAD_ARG;
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
