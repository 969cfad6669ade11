// Helpers of the mma.sync attention kernels: asynchronous 16-byte copies into shared
// memory, ldmatrix, the bf16 m16n8k16 tensor-core instruction, and the XOR swizzle of a
// [rows][D] bf16 tile that keeps ldmatrix free of bank conflicts.
#pragma once

#include "common.cuh"

namespace pb {

typedef __nv_bfloat16 bf16;

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Copies 16 bytes global -> shared without passing through registers; with pred false the
// 16 bytes are filled with zeros and the source is not read.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool pred) {
    const int bytes = pred ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
}
// The same copy with an L2 cache policy (from l2_policy_evict_first / l2_policy_normal).
__device__ __forceinline__ void cp_async16_policy(uint32_t dst, const void* src, bool pred, uint64_t policy) {
    const int bytes = pred ? 16 : 0;
    asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2, %3;\n" ::"r"(dst), "l"(src), "r"(bytes), "l"(policy));
}
// Lines fetched under this policy are the first to leave L2: for data that is read once per step and is larger than L2.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;\n" : "=l"(policy));
    return policy;
}
__device__ __forceinline__ uint64_t l2_policy_normal() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;\n" : "=l"(policy));
    return policy;
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// D (16x8, f32) += A (16x16, bf16, row) * B (16x8, bf16, col)
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Byte offset of 16-byte chunk `chunk` of row `row` in a [rows][D] bf16 tile.
template <int D>
__device__ __forceinline__ uint32_t tile_offset(int row, int chunk) {
    constexpr int kChunks = D / 8;
    return (uint32_t)(row * kChunks + (chunk ^ (row & 7))) * 16u;
}

// Gathers one 64-key tile of K and of V for kv head `kvh` through the block table into two
// swizzled shared-memory tiles with 16-byte asynchronous copies.  Keys outside
// [first_key, last_key] are filled with zeros and their pages are not touched.  Pages hold
// 2^page_shift keys (a power of two that divides 64); pools are [pages, Hkv, page, D].
// Each thread keeps one 16-byte column and walks down the rows, so that the swizzle and
// most of the address are loop constants.
// Asks L2 for the pages of one 64-key tile of K and of V for kv head `kvh` (one bulk prefetch per page and pool,
// issued by the first threads): a later load_kv_tile of the same tile then finds them there.  Pages without a key in
// [first_key, last_key] are not touched.
template <int D>
__device__ __forceinline__ void prefetch_kv_tile_l2(const bf16* __restrict__ k_pool, const bf16* __restrict__ v_pool,
                                                    const int* __restrict__ table, int key0, int first_key, int last_key, int kvh,
                                                    int Hkv, int page_shift, int tid, const PoolBounds bounds = PoolBounds{0, nullptr}) {
    const int pages = 64 >> page_shift;
    if (tid >= 2 * pages) return;
    const int pj = tid % pages;
    const int key = key0 + (pj << page_shift);
    if (key > last_key || key + (1 << page_shift) - 1 < first_key) return;
    const int page = table[key >> page_shift];
    if (!page_ok(page, bounds)) return;
    const size_t page_elems = (size_t)D << page_shift;
    const bf16* src = (tid < pages ? k_pool : v_pool) + (size_t)(page * Hkv + kvh) * page_elems;
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"((uint32_t)(page_elems * 2)) : "memory");
}

template <int D, int THREADS>
__device__ __forceinline__ void load_kv_tile(uint32_t k_dst, uint32_t v_dst, const bf16* __restrict__ k_pool,
                                             const bf16* __restrict__ v_pool, const int* __restrict__ table, int key0,
                                             int first_key, int last_key, int kvh, int Hkv, int page_shift, int tid,
                                             uint64_t policy = 0, const PoolBounds bounds = PoolBounds{0, nullptr}) {
    constexpr int kChunks = D / 8;
    constexpr int kRowsPerPass = THREADS / kChunks;       // a multiple of 8: (row & 7) does not change
    constexpr int kPasses = 64 / kRowsPerPass;
    static_assert(THREADS % kChunks == 0 && kRowsPerPass % 8 == 0 && 64 % kRowsPerPass == 0, "tile loader shape");
    const int c = tid % kChunks, r0 = tid / kChunks;
    const uint32_t off0 = tile_offset<D>(r0, c);
    const int page_mask = (1 << page_shift) - 1;
    const size_t page_elems = (size_t)D << page_shift;    // elements of one (page, kv head) block
    const int col = c * 8;
    if (key0 >= first_key && key0 + 63 <= last_key) {
#pragma unroll
        for (int i = 0; i < kPasses; ++i) {
            const int key = key0 + r0 + i * kRowsPerPass;
            int page = table[key >> page_shift];
            if (!page_ok(page, bounds)) page = 0;
            const size_t at = (size_t)(page * Hkv + kvh) * page_elems + (size_t)((key & page_mask) * D + col);
            const uint32_t off = off0 + (uint32_t)(i * kRowsPerPass * kChunks * 16);
            if (policy) {
                cp_async16_policy(k_dst + off, k_pool + at, true, policy);
                cp_async16_policy(v_dst + off, v_pool + at, true, policy);
            } else {
                cp_async16(k_dst + off, k_pool + at, true);
                cp_async16(v_dst + off, v_pool + at, true);
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < kPasses; ++i) {
            const int key = key0 + r0 + i * kRowsPerPass;
            const bool ok = key >= first_key && key <= last_key;
            size_t at = 0;
            if (ok) {
                int page = table[key >> page_shift];
                if (!page_ok(page, bounds)) page = 0;
                at = (size_t)(page * Hkv + kvh) * page_elems + (size_t)((key & page_mask) * D + col);
            }
            const uint32_t off = off0 + (uint32_t)(i * kRowsPerPass * kChunks * 16);
            if (policy) {
                cp_async16_policy(k_dst + off, k_pool + at, ok, policy);
                cp_async16_policy(v_dst + off, v_pool + at, ok, policy);
            } else {
                cp_async16(k_dst + off, k_pool + at, ok);
                cp_async16(v_dst + off, v_pool + at, ok);
            }
        }
    }
}

// log2 of a power of two (host side); -1 otherwise.
inline int log2_exact(int v) {
    if (v <= 0 || (v & (v - 1))) return -1;
    int s = 0;
    while ((1 << s) < v) ++s;
    return s;
}

}  // namespace pb
