// Sampling over rows of float32 logits, one block per row, each row with its own parameters.
//   greedy (top_k == 1 or temperature == 0): the largest logit, lowest index on ties;
//   otherwise: weights w_i = exp((l_i - max) / temperature); keep the top_k largest logits (ties
//   at the edge all kept; top_k <= 0: all), of those the smallest set of largest logits whose
//   weight reaches top_p of the kept weight (ties kept), then walk the kept tokens in index order
//   until the running weight passes u * (kept weight), u in [0,1) given per row.
// Thresholds are found by bisection over the order-preserving integer image of a float, with
// counts and sums reduced in a fixed order, so a row's result is reproducible and independent of
// the other rows.
#include "common.cuh"

#define SP_THREADS 1024

__device__ __forceinline__ unsigned sp_key(float x) {
    unsigned u = __float_as_uint(x);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ int sp_block_sum_int(int v, int* sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    int t = (lane < (SP_THREADS >> 5)) ? sh[lane] : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    return t;
}

__global__ void __launch_bounds__(SP_THREADS) sample_kernel(const float* __restrict__ logits, int ld, int V,
                                                            const float* __restrict__ temperature,
                                                            const int* __restrict__ top_k, const float* __restrict__ top_p,
                                                            const float* __restrict__ uniform, int* __restrict__ out) {
    __shared__ float shf[32];
    __shared__ int shi[32];
    __shared__ float s_prefix[SP_THREADS];
    __shared__ int s_result;
    il_pdl_begin();
    const int r = blockIdx.x, tid = threadIdx.x;
    const float* row = logits + (size_t)r * ld;

    // max and its lowest index
    float m = -INFINITY;
    int mi = 0x7fffffff;
    for (int i = tid; i < V; i += SP_THREADS) {
        const float x = row[i];
        if (x > m || (x == m && i < mi)) { m = x; mi = i; }
    }
    const float bm = il_block_max(m, shf);
    int cand = (m == bm) ? mi : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
    __syncthreads();
    if ((tid & 31) == 0) shi[tid >> 5] = cand;
    __syncthreads();
    int c2 = ((tid & 31) < (SP_THREADS >> 5)) ? shi[tid & 31] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) c2 = min(c2, __shfl_xor_sync(0xffffffffu, c2, o));
    const int arg = c2;

    const float T = temperature ? temperature[r] : 1.f;
    const int k = top_k ? top_k[r] : 0;
    const float pnuc = top_p ? top_p[r] : 1.f;
    if (k == 1 || T <= 0.f || !isfinite(bm)) {
        if (tid == 0) out[r] = arg;
        return;
    }
    const float invT = 1.f / T;

    // top-k: the largest key K with count(key >= K) >= k
    unsigned kth = 0u;
    if (k > 0 && k < V) {
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned tryk = kth | (1u << bit);
            int cnt = 0;
            for (int i = tid; i < V; i += SP_THREADS) cnt += sp_key(row[i]) >= tryk;
            cnt = sp_block_sum_int(cnt, shi);
            if (cnt >= k) kth = tryk;
        }
    }
    // kept weight after top-k
    float wk = 0.f;
    for (int i = tid; i < V; i += SP_THREADS) {
        const float x = row[i];
        if (sp_key(x) >= kth) wk += expf((x - bm) * invT);
    }
    wk = il_block_sum(wk, shf);
    // top-p: the largest key K >= kth with weight(key >= K) >= top_p * wk
    unsigned thr = kth;
    if (pnuc < 1.f) {
        const float target = pnuc * wk;
        unsigned K = 0u;
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned tryk = K | (1u << bit);
            float s = 0.f;
            for (int i = tid; i < V; i += SP_THREADS) {
                const float x = row[i];
                if (sp_key(x) >= tryk) s += expf((x - bm) * invT);
            }
            s = il_block_sum(s, shf);
            if (s >= target) K = tryk;
        }
        if (K > thr) thr = K;
    }
    // walk in index order: contiguous chunk per thread, exclusive scan over threads
    const int C = (V + SP_THREADS - 1) / SP_THREADS;
    const int i0 = tid * C, i1 = min(V, i0 + C);
    float mine = 0.f;
    for (int i = i0; i < i1; ++i) {
        const float x = row[i];
        if (sp_key(x) >= thr) mine += expf((x - bm) * invT);
    }
    s_prefix[tid] = mine;
    if (tid == 0) s_result = -1;
    __syncthreads();
    if (tid == 0) {  // serial scan: 1024 adds in a fixed order
        float run = 0.f;
        for (int t = 0; t < SP_THREADS; ++t) {
            const float v = s_prefix[t];
            s_prefix[t] = run;
            run += v;
        }
        shf[0] = run;
    }
    __syncthreads();
    const float total = shf[0];
    const float target = uniform[r] * total;
    const float before = s_prefix[tid];
    if (mine > 0.f && target >= before && target < before + mine) {
        float run = before;
        int pick = -1;
        for (int i = i0; i < i1; ++i) {
            const float x = row[i];
            if (sp_key(x) >= thr) {
                run += expf((x - bm) * invT);
                pick = i;
                if (run > target) break;
            }
        }
        s_result = pick;
    }
    __syncthreads();
    if (tid == 0) out[r] = s_result >= 0 ? s_result : arg;  // rounding at the far end: the mode
}

IL_EXPORT int il_sample(const float* logits, int ld, int R, int V, const float* temperature, const int* top_k,
                        const float* top_p, const float* uniform, int* out, cudaStream_t stream) {
    if (R <= 0) return IL_OK;
    if (V <= 0 || ld < V) return IL_BAD_ARG;
    IL_LAUNCH(sample_kernel, R, SP_THREADS, 0, stream, logits, ld, V, temperature, top_k, top_p, uniform, out);
    IL_LAUNCH_CHECK();
    return IL_OK;
}
