// out[M, N] = x[M, K] * W[N, K]^T for many tokens in bfloat16 on the fifth-generation tensor
// cores: tcgen05.mma with the accumulator in tensor memory, operands brought into shared
// memory by TMA (cp.async.bulk.tensor) and handed over through mbarriers.
//
// A persistent grid of one block per SM walks over tiles of 128 tokens x 256 features (token
// tiles fastest, so that blocks running together share one tile of W).  Roles inside a block:
//   warp 0, one thread   TMA producer: per 64-wide slice of K one [128 x 64] box of x and two
//                        [128 x 64] boxes of W into a 4-stage ring (128-byte swizzle), each
//                        stage guarded by a "full" barrier that counts the arriving bytes;
//   warp 1, one thread   MMA issuer: four tcgen05.mma (M 128, N 256, K 16) per stage straight
//                        from shared memory into one of two 256-column accumulators in tensor
//                        memory; a tcgen05.commit releases the stage ("empty" barrier) when the
//                        tensor core has read it, another announces the finished accumulator;
//   warps 2-5            epilogue: tcgen05.ld of the warp's 32 lanes (= 32 tokens), 32 columns
//                        at a time, rounding and store, while the MMA warp already fills the
//                        other accumulator with the next tile.
// Epilogues: plain (bfloat16 or float32), or SwiGLU: the 256 columns are 128 gate features and
// the 128 up features that belong to them (two TMA boxes from the two halves of the fused
// weight), and silu(gate) * up is written, so the [M, 2I] intermediate never exists.
//
// Rows of x or W beyond the matrix and the tail of K are zero-filled by TMA; stores are
// guarded.  Every wait is bounded by a clock limit: a block that gives up sets an error word
// that the host can read, lets its copies land, frees its tensor memory and returns.
//
// The reference calls at::linear (cuBLAS) for all of these (pulsar-core/src/model/qwen3.cpp:82-84,
// 114, 117-119) and two elementwise kernels for the gating.
#include "tcgen05_common.cuh"

#include <cstdlib>

namespace {

using namespace pb;
typedef __nv_bfloat16 bf16;

constexpr int kBM = 128;             // tokens per tile   (MMA M, TMEM lanes)
constexpr int kBN = 256;             // features per tile (MMA N, TMEM columns)
constexpr int kBK = 64;              // k per stage: one 128-byte swizzle atom of bfloat16
constexpr int kStages = 4;
constexpr int kThreads = 192;         // producer warp, MMA warp, four epilogue warps
constexpr int kAccumulators = 2;
constexpr int kTmemColumns = kAccumulators * kBN;   // all 512 columns of the SM's tensor memory
constexpr int kABytes = kBM * kBK * 2;           // 16 KB
constexpr int kBBytes = kBN * kBK * 2;           // 32 KB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kSmemBytes = kStages * kStageBytes + 1024 /* alignment slack */ + 256 /* barriers */;

enum { kPlain = 0, kSwiGLU = 1 };

__device__ unsigned int g_tc5_error = 0;          // 0 = fine; else 1 + the role that gave up

// Shared-memory matrix descriptor of a K-major tile with 128-byte rows and 128-byte swizzle:
// start address, leading offset 1 (unused by swizzled K-major layouts), 1024 bytes between
// groups of 8 rows, descriptor version 1, layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t umma_desc(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3fff);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Instruction descriptor: float32 accumulator, bfloat16 A and B, both K-major, N >> 3, M >> 4.
constexpr uint32_t kInstrDesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kBN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(kInstrDesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void store32(bf16* dst, const float (&f)[32], int n_valid) {
    if (n_valid >= 32 && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const __nv_bfloat162 v = __floats2bfloat162_rn(f[i * 8 + 2 * j], f[i * 8 + 2 * j + 1]);
                w[j] = *reinterpret_cast<const uint32_t*>(&v);
            }
            reinterpret_cast<uint4*>(dst)[i] = make_uint4(w[0], w[1], w[2], w[3]);
        }
    } else {
        for (int i = 0; i < 32 && i < n_valid; ++i) dst[i] = __float2bfloat16_rn(f[i]);
    }
}
__device__ __forceinline__ void store32(float* dst, const float (&f)[32], int n_valid) {
    if (n_valid >= 32 && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) reinterpret_cast<float4*>(dst)[i] = make_float4(f[4 * i], f[4 * i + 1], f[4 * i + 2], f[4 * i + 3]);
    } else {
        for (int i = 0; i < 32 && i < n_valid; ++i) dst[i] = f[i];
    }
}

// ---------------------------------------------------------------------------------------------
// The same product with pairs of blocks (a cluster of two on the two SMs of a TPC) working on a
// tile of 256 tokens x 256 features: tcgen05.mma.cta_group::2.  Each block of the pair loads its
// own 128 token rows of x and one half of the tile's 256 weight rows (so W crosses L2 -> shared
// memory once per pair, not once per block), and holds the accumulator of its own 128 tokens in
// its own tensor memory.  The block of rank 0 issues the MMAs for both.  Barriers:
//   full[s]       in rank 0, one arrival (rank 0's producer) that expects the bytes of both blocks;
//                 the TMA loads of both blocks complete their bytes on it;
//   empty[s]      in both blocks; released by a multicast tcgen05.commit when the MMAs have read it;
//   acc_full[a]   in both blocks; multicast commit after the tile's last MMA;
//   acc_empty[a]  in rank 0, eight arrivals: the four epilogue warps of each block.
// Shared-memory addresses of the two blocks differ in one bit (0x01000000) of the cluster window;
// clearing it turns a block's own barrier address into the address of rank 0's barrier.
constexpr uint32_t kPeerBitMask = 0xFEFFFFFFu;
constexpr int kPairStages = 6;
constexpr int kPairStageBytes = kABytes + kBBytes / 2;          // per block: 128 rows of x, 128 rows of W
constexpr int kPairSmemBytes = kPairStages * kPairStageBytes + 1024 + 256;
constexpr uint32_t kPairInstrDesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kBN >> 3) << 17) | ((uint32_t)((2 * kBM) >> 4) << 24);

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {            // `bar` is an address in the cluster window
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_rank0, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar_rank0), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(kPairInstrDesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {               // arrives on `bar` in both blocks
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((unsigned short)3) : "memory");
}

template <int MODE, typename OutT>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                         OutT* __restrict__ out, int M, int N, int K, int inter, int m_tiles, int n_tiles) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kPairStages * kPairStageBytes);   // full, empty, acc_full, acc_empty
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kPairStages + 2 * kAccumulators);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = cluster_rank();
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    constexpr int kTileCols = (MODE == kSwiGLU) ? kBN / 2 : kBN;
    const int k_tiles = (K + kBK - 1) / kBK;
    const int total_tiles = m_tiles * n_tiles;                  // m_tiles counts tiles of 256 tokens here
    const uint32_t full0 = smem_addr(bars), empty0 = smem_addr(bars + kPairStages);
    const uint32_t acc_full0 = smem_addr(bars + 2 * kPairStages), acc_empty0 = smem_addr(bars + 2 * kPairStages + kAccumulators);

    if (tid == 0) {
        for (int s = 0; s < kPairStages; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int a = 0; a < kAccumulators; ++a) { mbar_init(acc_full0 + 8 * a, 1); mbar_init(acc_empty0 + 8 * a, 8); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(kTmemColumns));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();                       // the peer's barriers exist before anything arrives on them
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer (in both blocks; bytes land on rank 0's full barrier)
        if (lane == 0) {
            uint32_t it = 0;
            for (int tile = pair; tile < total_tiles; tile += n_pairs) {
                const int m0 = (tile % m_tiles) * (2 * kBM) + (int)rank * kBM, n0 = (tile / m_tiles) * kTileCols;
                const int w_row = (MODE == kSwiGLU) ? (rank == 0 ? n0 : inter + n0) : n0 + (int)rank * (kBN / 2);
                bool ok = true;
                for (int kt = 0; kt < k_tiles; ++kt, ++it) {
                    const int s = it % kPairStages;
                    if (!mbar_wait(empty0 + 8 * s, ((it / kPairStages) & 1) ^ 1, abort_flag)) { ok = false; break; }
                    const uint32_t a_dst = smem_addr(smem + s * kPairStageBytes), b_dst = a_dst + kABytes;
                    const uint32_t full_rank0 = (full0 + 8 * s) & kPeerBitMask;
                    if (rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * kPairStageBytes);
                    tma_load_2d_pair(a_dst, &map_x, full_rank0, kt * kBK, m0);
                    tma_load_2d_pair(b_dst, &map_w, full_rank0, kt * kBK, w_row);
                }
                if (!ok) { *abort_flag = 1; atomicMax(&g_tc5_error, 2u); break; }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: rank 0 only, for both blocks.  The whole warp walks the loop and waits on the
        // barriers, one elected lane issues: with uniform control flow the descriptors live in uniform registers and
        // the issuing stream is short (an MMA is accepted only when the one before it has started, so every cycle
        // that the issuing lane needs beyond an MMA's own time is a cycle without products).
        if (rank == 0) {
            const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);         // (a broadcast: uniform for the compiler)
            const uint64_t desc0 = umma_desc(smem_addr(smem));
            uint32_t it = 0;
            int j = 0;
            bool ok = true;
            for (int tile = pair; tile < total_tiles && ok; tile += n_pairs, ++j) {
                const int acc = j & 1;
                ok = mbar_wait(acc_empty0 + 8 * acc, ((j >> 1) & 1) ^ 1, abort_flag);
                const uint32_t tmem_d = tmem_u + acc * kBN;
                for (int kt = 0; kt < k_tiles && ok; ++kt, ++it) {
                    const int s = it % kPairStages;
                    if (!mbar_wait(full0 + 8 * s, (it / kPairStages) & 1, abort_flag)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    // descriptors differ from stage to stage only in their address field (16-byte units)
                    const uint64_t a_desc = desc0 + (uint64_t)((uint32_t)s * (kPairStageBytes >> 4));
                    const uint64_t b_desc = a_desc + (uint64_t)(kABytes >> 4);
                    if (elect_one()) {
#pragma unroll
                        for (int k = 0; k < kBK / 16; ++k)
                            umma_bf16_pair(tmem_d, a_desc + (uint64_t)(k * 2), b_desc + (uint64_t)(k * 2), (kt > 0 || k > 0) ? 1u : 0u);
                        umma_commit_pair(empty0 + 8 * s);
                        if (kt == k_tiles - 1) umma_commit_pair(acc_full0 + 8 * acc);
                    }
                    __syncwarp();
                }
            }
            if (!ok && lane == 0) { *abort_flag = 1; atomicMax(&g_tc5_error, 3u); }
        }
    } else {
        // ---------------- epilogue of this block's 128 tokens
        const int quarter = warp & 3;
        int j = 0;
        for (int tile = pair; tile < total_tiles; tile += n_pairs, ++j) {
            const int acc = j & 1;
            const int m0 = (tile % m_tiles) * (2 * kBM) + (int)rank * kBM, n0 = (tile / m_tiles) * kTileCols;
            if (!mbar_wait(acc_full0 + 8 * acc, (j >> 1) & 1, abort_flag)) {
                if (lane == 0) { *abort_flag = 1; atomicMax(&g_tc5_error, 4u); }
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int row = m0 + quarter * 32 + lane;
            const uint32_t lane_base = tmem_base + acc * kBN + ((uint32_t)(quarter * 32) << 16);
            if (MODE == kSwiGLU) {
#pragma unroll 1
                for (int c = 0; c < kBN / 2; c += 32) {
                    uint32_t gv[32], uv[32];
                    tmem_ld32(lane_base + c, gv);
                    tmem_ld32(lane_base + kBN / 2 + c, uv);
                    float f[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const float g = __uint_as_float(gv[i]), u = __uint_as_float(uv[i]);
                        f[i] = g / (1.0f + expf(-g)) * u;
                    }
                    if (row < M && n0 + c < inter) store32(out + (size_t)row * inter + n0 + c, f, inter - (n0 + c));
                }
            } else {
#pragma unroll 1
                for (int c = 0; c < kBN; c += 32) {
                    uint32_t v[32];
                    tmem_ld32(lane_base + c, v);
                    float f[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(v[i]);
                    if (row < M && n0 + c < N) store32(out + (size_t)row * N + n0 + c, f, N - (n0 + c));
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster((acc_empty0 + 8 * acc) & kPeerBitMask);
        }
    }
    __syncwarp();
    if (*abort_flag) {
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();                       // neither block leaves while the other may still touch its memory
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemColumns));
}

// Tiles are numbered with the token tile fastest; block b takes tiles b, b + gridDim.x, ...
// Plain: W rows [n0, n0 + 256) of N.  SwiGLU: gate rows [g0, g0 + 128) and up rows [inter + g0, ...): the output
// has `inter` columns and a tile covers 128 of them.
template <int MODE, typename OutT>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    OutT* __restrict__ out, int M, int N, int K, int inter, int m_tiles, int n_tiles) {
    extern __shared__ unsigned char smem_raw[];
    // 128-byte swizzled tiles want 1024-byte alignment.
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);   // full[4], empty[4], acc_full[2], acc_empty[2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 2 * kAccumulators);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    constexpr int kTileCols = (MODE == kSwiGLU) ? kBN / 2 : kBN;        // output columns of a tile
    const int k_tiles = (K + kBK - 1) / kBK;
    const int total_tiles = m_tiles * n_tiles;
    const uint32_t full0 = smem_addr(bars), empty0 = smem_addr(bars + kStages);
    const uint32_t acc_full0 = smem_addr(bars + 2 * kStages), acc_empty0 = smem_addr(bars + 2 * kStages + kAccumulators);

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int a = 0; a < kAccumulators; ++a) { mbar_init(acc_full0 + 8 * a, 1); mbar_init(acc_empty0 + 8 * a, 4); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {            // one warp allocates the accumulator columns and keeps the right to free them
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(kTmemColumns));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer
        if (lane == 0) {
            uint32_t it = 0;                                  // k-slices issued so far, over all tiles
            for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
                const int m0 = (tile % m_tiles) * kBM, n0 = (tile / m_tiles) * kTileCols;
                bool ok = true;
                for (int kt = 0; kt < k_tiles; ++kt, ++it) {
                    const int s = it % kStages;
                    if (!mbar_wait(empty0 + 8 * s, ((it / kStages) & 1) ^ 1, abort_flag)) { ok = false; break; }
                    const uint32_t a_dst = smem_addr(smem + s * kStageBytes), b_dst = a_dst + kABytes;
                    mbar_expect_tx(full0 + 8 * s, kStageBytes);
                    tma_load_2d(a_dst, &map_x, full0 + 8 * s, kt * kBK, m0);
                    tma_load_2d(b_dst, &map_w, full0 + 8 * s, kt * kBK, n0);
                    tma_load_2d(b_dst + kBBytes / 2, &map_w, full0 + 8 * s, kt * kBK, (MODE == kSwiGLU ? inter : kBN / 2) + n0);
                }
                if (!ok) { *abort_flag = 1; atomicMax(&g_tc5_error, 2u); break; }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: the warp walks the loop uniformly, one elected lane issues
        {
            const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
            const uint64_t desc0 = umma_desc(smem_addr(smem));
            uint32_t it = 0;
            int j = 0;                                        // tiles done by this block
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++j) {
                const int acc = j & 1;
                ok = mbar_wait(acc_empty0 + 8 * acc, ((j >> 1) & 1) ^ 1, abort_flag);   // the epilogue has drained it
                const uint32_t tmem_d = tmem_u + acc * kBN;
                for (int kt = 0; kt < k_tiles && ok; ++kt, ++it) {
                    const int s = it % kStages;
                    if (!mbar_wait(full0 + 8 * s, (it / kStages) & 1, abort_flag)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t a_desc = desc0 + (uint64_t)((uint32_t)s * (kStageBytes >> 4));
                    const uint64_t b_desc = a_desc + (uint64_t)(kABytes >> 4);
                    if (elect_one()) {
#pragma unroll
                        for (int k = 0; k < kBK / 16; ++k)      // 16 bfloat16 = 32 bytes further along the 128-byte row
                            umma_bf16(tmem_d, a_desc + (uint64_t)(k * 2), b_desc + (uint64_t)(k * 2), (kt > 0 || k > 0) ? 1u : 0u);
                        umma_commit(empty0 + 8 * s);          // the stage is free once the tensor core has read it
                        if (kt == k_tiles - 1) umma_commit(acc_full0 + 8 * acc);     // the accumulator is complete once its MMAs have retired
                    }
                    __syncwarp();
                }
            }
            if (!ok && lane == 0) { *abort_flag = 1; atomicMax(&g_tc5_error, 3u); }
        }
    } else {
        // ---------------- epilogue: warp w reads the lanes of tensor memory it may touch (32 * (w % 4) ...)
        const int quarter = warp & 3;
        int j = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++j) {
            const int acc = j & 1;
            const int m0 = (tile % m_tiles) * kBM, n0 = (tile / m_tiles) * kTileCols;
            if (!mbar_wait(acc_full0 + 8 * acc, (j >> 1) & 1, abort_flag)) {
                if (lane == 0) { *abort_flag = 1; atomicMax(&g_tc5_error, 4u); }
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int row = m0 + quarter * 32 + lane;
            const uint32_t lane_base = tmem_base + acc * kBN + ((uint32_t)(quarter * 32) << 16);
            if (MODE == kSwiGLU) {
#pragma unroll 1
                for (int c = 0; c < kBN / 2; c += 32) {
                    uint32_t gv[32], uv[32];
                    tmem_ld32(lane_base + c, gv);
                    tmem_ld32(lane_base + kBN / 2 + c, uv);
                    float f[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const float g = __uint_as_float(gv[i]), u = __uint_as_float(uv[i]);
                        f[i] = g / (1.0f + expf(-g)) * u;
                    }
                    if (row < M && n0 + c < inter) store32(out + (size_t)row * inter + n0 + c, f, inter - (n0 + c));
                }
            } else {
#pragma unroll 1
                for (int c = 0; c < kBN; c += 32) {
                    uint32_t v[32];
                    tmem_ld32(lane_base + c, v);
                    float f[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(v[i]);
                    if (row < M && n0 + c < N) store32(out + (size_t)row * N + n0 + c, f, N - (n0 + c));
                }
            }
            // this warp has read its part of the accumulator: one of the four arrivals that free it
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty0 + 8 * acc);
        }
    }
    __syncwarp();
    if (*abort_flag) {
        // a role gave up: give copies that are still in flight time to land before this block's memory is reused
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemColumns));
}

// Row-major [rows, K] bfloat16 matrix, boxes of 128 rows x 64 columns, 128-byte swizzle, zero fill outside.
int make_map(CUtensorMap* map, const void* base, int rows, int K) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return (int)cudaErrorNotSupported;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {kBK, 128};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult rc = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return rc == CUDA_SUCCESS ? 0 : PB_ERR_BAD_SIZE;
}

bool pair_enabled() {      // PULSAR_TCGEN05_PAIR=0 keeps every product on single blocks
    static const bool on = [] {
        const char* v = getenv("PULSAR_TCGEN05_PAIR");
        return !(v && v[0] == '0' && v[1] == 0);
    }();
    return on;
}

int sm_count() {
    static int n = [] {
        int dev = 0, v = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) v = 0;
        return v > 0 ? v : 148;
    }();
    return n;
}

template <int MODE, typename OutT>
int launch(const CUtensorMap& mx, const CUtensorMap& mw, void* out, int M, int N, int K, int inter, int m_tiles, int n_tiles,
           cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        cudaError_t rc = cudaFuncSetAttribute(gemm_tcgen05_kernel<MODE, OutT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (rc != cudaSuccess) return (int)rc;
        configured = true;
    }
    if (M > kBM && pair_enabled()) {
        // more than one tile of tokens: pairs of blocks on tiles of 256 tokens
        static bool pair_configured = false;
        if (!pair_configured) {
            cudaError_t rc = cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<MODE, OutT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmemBytes);
            if (rc != cudaSuccess) return (int)rc;
            pair_configured = true;
        }
        const int pm_tiles = (M + 2 * kBM - 1) / (2 * kBM);
        const long long ptiles = (long long)pm_tiles * n_tiles;
        const int pairs = (int)(ptiles < sm_count() / 2 ? ptiles : sm_count() / 2);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * pairs);
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = kPairSmemBytes;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        return (int)cudaLaunchKernelEx(&cfg, gemm_tcgen05_pair_kernel<MODE, OutT>, mx, mw, (OutT*)out, M, N, K, inter, pm_tiles, n_tiles);
    }
    const long long tiles = (long long)m_tiles * n_tiles;
    const int grid = (int)(tiles < sm_count() ? tiles : sm_count());       // persistent: one block per SM
    gemm_tcgen05_kernel<MODE, OutT><<<grid, kThreads, kSmemBytes, stream>>>(mx, mw, (OutT*)out, M, N, K, inter, m_tiles, n_tiles);
    return launch_status();
}

}  // namespace

// 1 if pb_gemm_tcgen05 takes this problem: K a multiple of 8 (TMA strides are multiples of 16 bytes);
// SwiGLU additionally needs the gate/up halves to split evenly.
PB_EXPORT int pb_gemm_tcgen05_supported(int mode, int M, int N, int K) {
    if (M <= 0 || N <= 0 || K <= 0 || (K % 8)) return 0;
    if (mode == kSwiGLU) return (N % 2 == 0) ? 1 : 0;
    return mode == kPlain ? 1 : 0;
}

// The error word of the kernel's bounded waits (0 = no block ever gave up); reading it synchronises.
PB_EXPORT int pb_gemm_tcgen05_error(void) {
    unsigned int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc5_error, sizeof(v)) != cudaSuccess) return -1;
    return (int)v;
}

// limit > 0: the new limit of the kernel's bounded waits in clock cycles; error >= 0: the new value of the error
// word; address: receives the word's device address.  Returns 0, or -1 when a CUDA call failed.
PB_EXPORT int pb_gemm_tcgen05_wait_control(long long limit, int error, void** address) {
    return wait_control(g_tc5_error, limit, error, address);
}

namespace {
// One thread waits, with the limit of the bounded waits, on a barrier that nobody arrives on, gives up and sets the
// error word: the give-up path of the kernels above, alone (no copy in flight, no tensor memory held).
__global__ void wait_selftest_kernel() {
    __shared__ __align__(8) uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(smem_addr(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (!mbar_wait(smem_addr(&bar), 0, &abort_flag)) {
            abort_flag = 1;
            atomicMax(&g_tc5_error, 9u);
        }
        asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_addr(&bar)) : "memory");
    }
}
}  // namespace

// Runs the kernel above: afterwards the error word reads 9.  With the first limit it takes about two seconds;
// set a short limit first.
PB_EXPORT int pb_gemm_tcgen05_wait_selftest(cudaStream_t stream) {
    wait_selftest_kernel<<<1, 32, 0, stream>>>();
    return launch_status();
}

// mode 0: out[M, N] = x W^T (out_dtype bfloat16 or float32).  mode 1: W = [gate rows; up rows], N = 2 * inter,
// out[M, inter] = silu(x Wg^T) * (x Wu^T) in bfloat16.  x [M, K] and W [N, K] bfloat16, 16-byte aligned.
PB_EXPORT int pb_gemm_tcgen05(int mode, int out_dtype, const void* x, const void* w, void* out, int M, int N, int K,
                              cudaStream_t stream) {
    if (!pb_gemm_tcgen05_supported(mode, M, N, K)) return PB_ERR_BAD_SIZE;
    if ((((uintptr_t)x | (uintptr_t)w) & 15) != 0) return PB_ERR_BAD_SIZE;
    if (out_dtype != PB_BF16 && out_dtype != PB_F32) return PB_ERR_BAD_DTYPE;
    CUtensorMap mx, mw;
    int rc = make_map(&mx, x, M, K);
    if (rc != 0) return rc;
    rc = make_map(&mw, w, N, K);
    if (rc != 0) return rc;
    const int m_tiles = (M + kBM - 1) / kBM;
    if (mode == kSwiGLU) {
        if (out_dtype != PB_BF16) return PB_ERR_BAD_DTYPE;
        const int inter = N / 2;
        return launch<kSwiGLU, bf16>(mx, mw, out, M, N, K, inter, m_tiles, (inter + kBN / 2 - 1) / (kBN / 2), stream);
    }
    const int n_tiles = (N + kBN - 1) / kBN;
    if (out_dtype == PB_BF16) return launch<kPlain, bf16>(mx, mw, out, M, N, K, 0, m_tiles, n_tiles, stream);
    return launch<kPlain, float>(mx, mw, out, M, N, K, 0, m_tiles, n_tiles, stream);
}
