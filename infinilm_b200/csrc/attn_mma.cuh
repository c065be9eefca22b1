// Building blocks of the bfloat16 attention kernels: asynchronous copies of cache pages into
// padded shared-memory tiles, ldmatrix fragment loads and the m16n8k16 tensor-core product
// with float32 accumulation.
//
// A tile row holds head_dim bfloat16 plus 16 bytes of padding, so that the eight 16-byte rows an
// ldmatrix reads fall into different bank groups for every head_dim that is a multiple of 16.
#pragma once
#include "common.cuh"

#ifndef HEAD_DIM
#error "compile with -DHEAD_DIM=<multiple of 16, 16..256>"
#endif
static_assert(HEAD_DIM % 16 == 0 && HEAD_DIM >= 16 && HEAD_DIM <= 256, "head_dim must be a multiple of 16 in [16,256]");

constexpr int AT_HD = HEAD_DIM;
constexpr int AT_ROW_BYTES = HEAD_DIM * 2 + 16;   // padded row of a K or V tile
constexpr int AT_CHUNKS = HEAD_DIM / 8;            // 16-byte chunks of a row
constexpr int AT_KSTEPS = HEAD_DIM / 16;           // k-steps of Q.K^T
constexpr int AT_NT = HEAD_DIM / 8;                // n-tiles of P.V

__device__ __forceinline__ void at_cp_async16(uint32_t smem_addr, const void* gptr) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_addr), "l"(gptr));
}
__device__ __forceinline__ void at_cp_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void at_cp_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void at_ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void at_ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
// D(16x8, f32) += A(16x16, bf16 row-major) * B(16x8, bf16 col-major)
__device__ __forceinline__ void at_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t at_pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Copies `n_keys` (<= 16, a page or its valid head) rows of one kv head's K and V from a cache page into tiles.
// page_base points at the page: [2][kv heads][page_size][head_dim]. One warp issues the copies.
__device__ __forceinline__ void at_load_page(uint32_t k_tile, uint32_t v_tile, const __nv_bfloat16* page_base, int g, int nkv,
                                             int page_size, int first_row, int n_rows, int lane) {
    const __nv_bfloat16* ksrc = page_base + ((size_t)g * page_size + first_row) * AT_HD;
    const __nv_bfloat16* vsrc = ksrc + (size_t)nkv * page_size * AT_HD;
    const int total = n_rows * AT_CHUNKS;
    for (int c = lane; c < total; c += 32) {
        const int r = c / AT_CHUNKS, cc = c - r * AT_CHUNKS;
        at_cp_async16(k_tile + r * AT_ROW_BYTES + cc * 16, ksrc + (size_t)r * AT_HD + cc * 8);
        at_cp_async16(v_tile + r * AT_ROW_BYTES + cc * 16, vsrc + (size_t)r * AT_HD + cc * 8);
    }
}

// S(16 rows x 16 keys) = Q . K^T for the 16 keys of a tile at `k_tile`; s[0] holds keys 0-7, s[1] keys 8-15.
__device__ __forceinline__ void at_qk_16keys(float (&s)[2][4], const uint32_t (&qf)[AT_KSTEPS][4], uint32_t k_tile, int lane) {
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
    const int mat = lane >> 3, r = lane & 7;
    const uint32_t base = k_tile + ((mat >> 1) * 8 + r) * AT_ROW_BYTES + (mat & 1) * 16;
#pragma unroll
    for (int kk = 0; kk < AT_KSTEPS; ++kk) {
        uint32_t b0, b1, b2, b3;
        at_ldmatrix_x4(b0, b1, b2, b3, base + kk * 32);
        at_mma(s[0], qf[kk], b0, b1);
        at_mma(s[1], qf[kk], b2, b3);
    }
}

// O(16 rows x head_dim) += P(16 rows x 16 keys) . V(16 keys x head_dim); pf is P as an A fragment.
__device__ __forceinline__ void at_pv_16keys(float (&o)[AT_NT][4], const uint32_t (&pf)[4], uint32_t v_tile, int lane) {
    const int mat = lane >> 3, r = lane & 7;
    const uint32_t base = v_tile + ((mat & 1) * 8 + r) * AT_ROW_BYTES + (mat >> 1) * 16;
#pragma unroll
    for (int nt = 0; nt < AT_NT; nt += 2) {
        uint32_t b0, b1, b2, b3;
        at_ldmatrix_x4_trans(b0, b1, b2, b3, base + nt * 16);
        at_mma(o[nt], pf, b0, b1);
        at_mma(o[nt + 1], pf, b2, b3);
    }
}

// Q rows as A fragments straight from global memory. row_ptr(r) gives the address of row r's
// head_dim bfloat16 (nullptr: a padding row of zeros).
template <typename RowPtr>
__device__ __forceinline__ void at_load_q(uint32_t (&qf)[AT_KSTEPS][4], RowPtr row_ptr, int lane) {
    const __nv_bfloat16* r0 = row_ptr(lane >> 2);
    const __nv_bfloat16* r1 = row_ptr((lane >> 2) + 8);
    const int c = (lane & 3) * 2;
#pragma unroll
    for (int kk = 0; kk < AT_KSTEPS; ++kk) {
        qf[kk][0] = r0 ? *reinterpret_cast<const uint32_t*>(r0 + kk * 16 + c) : 0u;
        qf[kk][1] = r1 ? *reinterpret_cast<const uint32_t*>(r1 + kk * 16 + c) : 0u;
        qf[kk][2] = r0 ? *reinterpret_cast<const uint32_t*>(r0 + kk * 16 + c + 8) : 0u;
        qf[kk][3] = r1 ? *reinterpret_cast<const uint32_t*>(r1 + kk * 16 + c + 8) : 0u;
    }
}
