// out[M, N] = x[M, K] * W[N, K]^T for 17 to 128 tokens in bfloat16: the projections of a decode step with
// dozens of sequences, where every weight is still read once and the time is the time to stream W from HBM,
// but there are too many tokens for the kernel that keeps them in MMA fragments (gemm_skinny.cu).
//
// The operands change places against gemm_tcgen05.cu: 128 rows of W are the 128-row operand of tcgen05.mma
// (the lanes of the accumulator in tensor memory), the tokens are its narrow one (16 to 128 columns).  A block
// owns one tile of 128 weight rows and a slice of K; the S blocks of a cluster own the S slices of one tile,
// so that a product with few tiles (4096 output features are 32 tiles) still has a block on nearly every SM
// and each block streams its part of W through a ring of TMA stages without a pause.  The partial sums meet
// in shared memory: every block of the cluster sends, for each token, its 128 partial sums to the block that
// owns that token's column slice (st.shared::cluster), one cluster barrier, and every block adds up and
// stores its own columns.  No partial sum goes through global memory, no atomics, a fixed order of addition.
//
// Roles in a block (192 threads): warp 0 / one thread issues the TMA loads (W with an evict-first L2 hint:
// weights are read once per step and are far larger than L2; W of the first stages is asked for before the
// kernel waits for its predecessor, x after), warp 1 / one thread issues the MMAs, warps 2-5 read the
// accumulator.  SwiGLU: a tile is 64 gate rows and the 64 up rows that belong to them (two TMA boxes), and
// silu(gate) * up is applied after the sums are complete, so the [M, 2I] intermediate never exists.
//
// Every wait on a barrier is bounded by a clock limit; a role that gives up sets the error word and every
// role still reaches the cluster barrier and frees the tensor memory.  No TMA load uses cluster multicast.
//
// The reference calls at::linear (cuBLAS) for all of these (pulsar-core/src/model/qwen3.cpp:82-84, 114, 117-119).
#include "tcgen05_common.cuh"

#include <cstdlib>

namespace {

using namespace pb;
typedef __nv_bfloat16 bf16;

constexpr int kRows = 128;            // weight rows per tile (MMA M, lanes of tensor memory)
constexpr int kBK = 64;               // k per stage: one 128-byte swizzle atom of bfloat16
constexpr int kThreads = 192;
constexpr int kWBytes = kRows * kBK * 2;      // 16 KB
constexpr int kTmemColumns = 128;
constexpr int kMaxStages = 8;
constexpr int kMaxCluster = 8;

enum { kPlain = 0, kSwiGLU = 1 };

__device__ unsigned int g_stream_error = 0;       // 0 = fine; else 1 + the role that gave up


__device__ __forceinline__ uint64_t umma_desc(uint32_t addr) {      // K-major, 128-byte rows, 128-byte swizzle
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3fff);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, uint64_t policy) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "l"(policy) : "memory");
}
__device__ __forceinline__ uint64_t policy_evict_first() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t remote_addr(uint32_t local, uint32_t rank) {      // the same offset in block `rank`'s shared memory
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
__device__ __forceinline__ void store_remote(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}

struct StreamArgs {
    int M, N, K, inter;
    int n_pad;          // tokens rounded up to a multiple of 16: columns of the accumulator, rows of an x box
    int stages;         // TMA stages of the ring
    int splits;         // blocks per cluster = slices of K
    int cols_per;       // token columns that a block of the cluster adds up and stores: ceil(M / splits)
    int recv_offset;    // bytes from the ring's start to the receive buffer (0: it takes the ring's place, splits == 1)
    int bar_offset;     // bytes from the ring's start to the barriers
};

template <int MODE, typename OutT>
__global__ void __launch_bounds__(kThreads)
gemm_tcgen05_stream_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                           OutT* __restrict__ out, const StreamArgs a) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int x_bytes = a.n_pad * kBK * 2;
    const int stage_bytes = kWBytes + x_bytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + a.bar_offset);            // full[stages], empty[stages], acc_full
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kMaxStages + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* recv = reinterpret_cast<float*>(smem + a.recv_offset);                 // [splits][cols_per][128]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = cluster_rank();
    const int tile = blockIdx.x / a.splits;
    const int k_tiles = (a.K + kBK - 1) / kBK;
    const int kt_begin = (int)((long long)k_tiles * rank / a.splits), kt_end = (int)((long long)k_tiles * (rank + 1) / a.splits);
    const int n_kt = kt_end - kt_begin;
    constexpr int kTileCols = (MODE == kSwiGLU) ? kRows / 2 : kRows;              // output features of a tile
    const int n0 = tile * kTileCols;
    const uint32_t full0 = smem_addr(bars), empty0 = smem_addr(bars + kMaxStages), acc_full = smem_addr(bars + 2 * kMaxStages);

    if (tid == 0) {
        for (int s = 0; s < a.stages; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        mbar_init(acc_full, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
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
            const uint64_t policy = policy_evict_first();
            auto load_w = [&](int s, int kt) {
                const uint32_t w_dst = smem_addr(smem + s * stage_bytes);
                mbar_expect_tx(full0 + 8 * s, stage_bytes);
                if (MODE == kSwiGLU) {
                    tma_load_2d_hint(w_dst, &map_w, full0 + 8 * s, kt * kBK, n0, policy);
                    tma_load_2d_hint(w_dst + kWBytes / 2, &map_w, full0 + 8 * s, kt * kBK, a.inter + n0, policy);
                } else {
                    tma_load_2d_hint(w_dst, &map_w, full0 + 8 * s, kt * kBK, n0, policy);
                }
            };
            auto load_x = [&](int s, int kt) {
                tma_load_2d(smem_addr(smem + s * stage_bytes + kWBytes), &map_x, full0 + 8 * s, kt * kBK, 0);
            };
            // the weights depend on no earlier kernel: the first stages' W is on its way before this kernel may read x
            const int first = n_kt < a.stages ? n_kt : a.stages;
            for (int i = 0; i < first; ++i) load_w(i, kt_begin + i);
            pdl_wait();
            for (int i = 0; i < first; ++i) load_x(i, kt_begin + i);
            bool ok = true;
            for (int i = first; i < n_kt; ++i) {
                const int s = i % a.stages;
                if (!mbar_wait(empty0 + 8 * s, ((i / a.stages) & 1) ^ 1, abort_flag)) { ok = false; break; }
                load_w(s, kt_begin + i);
                load_x(s, kt_begin + i);
            }
            if (!ok) { *abort_flag = 1; atomicMax(&g_stream_error, 2u); }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: the warp walks the loop uniformly, one elected lane issues
        const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
        const uint64_t desc0 = umma_desc(smem_addr(smem));
        // float32 accumulator, bfloat16 A and B, both K-major, N >> 3, M >> 4
        const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(a.n_pad >> 3) << 17) | ((uint32_t)(kRows >> 4) << 24);
        bool ok = true;
        for (int i = 0; i < n_kt; ++i) {
            const int s = i % a.stages;
            if (!mbar_wait(full0 + 8 * s, (i / a.stages) & 1, abort_flag)) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t w_desc = desc0 + (uint64_t)((uint32_t)(s * stage_bytes) >> 4);
            const uint64_t x_desc = w_desc + (uint64_t)(kWBytes >> 4);
            if (elect_one()) {
#pragma unroll
                for (int k = 0; k < kBK / 16; ++k)
                    umma_bf16(tmem_u, w_desc + (uint64_t)(k * 2), x_desc + (uint64_t)(k * 2), idesc, (i > 0 || k > 0) ? 1u : 0u);
                umma_commit(empty0 + 8 * s);
                if (i == n_kt - 1) umma_commit(acc_full);
            }
            __syncwarp();
        }
        if (!ok && lane == 0) { *abort_flag = 1; atomicMax(&g_stream_error, 3u); }
    } else {
        // ---------------- accumulator -> the blocks that own the token columns.  This thread holds weight row `row`.
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        bool ok = n_kt == 0 || mbar_wait(acc_full, 0, abort_flag);
        if (!ok && lane == 0) { *abort_flag = 1; atomicMax(&g_stream_error, 4u); }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        pdl_trigger();
        const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const uint32_t recv_local = smem_addr(recv);
        for (int c0 = 0; c0 < a.M; c0 += 32) {
            uint32_t v[32];
            if (ok && n_kt > 0) {
                tmem_ld32(lane_base + c0, v);
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = 0u;
            }
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const int c = c0 + i;
                if (c < a.M) {
                    const uint32_t owner = (uint32_t)(c / a.cols_per);
                    const uint32_t local = recv_local + (uint32_t)((((int)rank * a.cols_per + (c - (int)owner * a.cols_per)) * kRows + row) * 4);
                    if (a.splits == 1) *reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(recv) + (local - recv_local)) = __uint_as_float(v[i]);
                    else store_remote(remote_addr(local, owner), __uint_as_float(v[i]));
                }
            }
        }
    }
    __syncwarp();
    if (*abort_flag) {
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);      // copies that are still in flight may land
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();          // every block's partial sums have arrived; nobody writes into a peer's memory after this
    if (warp >= 2) {
        // ---------------- add up the slices of K for this block's token columns and store them
        const int r = (warp - 2) * 32 + lane;                  // weight row within the tile
        const int c_begin = (int)rank * a.cols_per;
        const int c_end = min(a.M, c_begin + a.cols_per);
        for (int c = c_begin; c < c_end; ++c) {
            const float* col = recv + (size_t)(c - c_begin) * kRows;
            if (MODE == kSwiGLU) {
                if (r < kRows / 2) {
                    float gate = 0.0f, up = 0.0f;
                    for (int s = 0; s < a.splits; ++s) {
                        gate += col[(size_t)s * a.cols_per * kRows + r];
                        up += col[(size_t)s * a.cols_per * kRows + r + kRows / 2];
                    }
                    if (n0 + r < a.inter) out[(size_t)c * a.inter + n0 + r] = from_float<OutT>(gate / (1.0f + expf(-gate)) * up);
                }
            } else {
                float sum = 0.0f;
                for (int s = 0; s < a.splits; ++s) sum += col[(size_t)s * a.cols_per * kRows + r];
                if (n0 + r < a.N) out[(size_t)c * a.N + n0 + r] = from_float<OutT>(sum);
            }
        }
    }
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemColumns));
}

// ---------------------------------------------------------------------------------------------
// The same product without slices of K, for weights with more tiles than SMs (gate/up, the head): a persistent
// grid of one block per SM walks over the tiles; two accumulators in tensor memory take turns, so that the ring of
// TMA stages never pauses while a finished tile is read out and stored.  Plain tiles are stored straight from
// registers (a warp's 32 lanes are 32 consecutive output features of one token); SwiGLU tiles pass the up half
// through shared memory to the warps that hold the gate half.
constexpr int kPersistTmem = 256;          // two accumulators of up to 128 columns

__device__ __forceinline__ void named_barrier(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

template <int MODE, typename OutT>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_stream_persistent_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                                      OutT* __restrict__ out, const StreamArgs a, int n_tiles) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int x_bytes = a.n_pad * kBK * 2;
    const int stage_bytes = kWBytes + x_bytes;
    float* stage_up = reinterpret_cast<float*>(smem + a.recv_offset);             // SwiGLU: [32 columns][64 rows]
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + a.bar_offset);            // full[8], empty[8], acc_full[2], acc_empty[2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kMaxStages + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int k_tiles = (a.K + kBK - 1) / kBK;
    constexpr int kTileCols = (MODE == kSwiGLU) ? kRows / 2 : kRows;
    const uint32_t full0 = smem_addr(bars), empty0 = smem_addr(bars + kMaxStages);
    const uint32_t acc_full0 = smem_addr(bars + 2 * kMaxStages), acc_empty0 = smem_addr(bars + 2 * kMaxStages + 2);

    if (tid == 0) {
        for (int s = 0; s < a.stages; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(acc_full0 + 8 * i, 1); mbar_init(acc_empty0 + 8 * i, 4); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(kPersistTmem));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer
        if (lane == 0) {
            const uint64_t policy = policy_evict_first();
            auto load_w = [&](int s, int kt, int n0) {
                const uint32_t w_dst = smem_addr(smem + s * stage_bytes);
                mbar_expect_tx(full0 + 8 * s, stage_bytes);
                tma_load_2d_hint(w_dst, &map_w, full0 + 8 * s, kt * kBK, n0, policy);
                if (MODE == kSwiGLU) tma_load_2d_hint(w_dst + kWBytes / 2, &map_w, full0 + 8 * s, kt * kBK, a.inter + n0, policy);
            };
            auto load_x = [&](int s, int kt) {
                tma_load_2d(smem_addr(smem + s * stage_bytes + kWBytes), &map_x, full0 + 8 * s, kt * kBK, 0);
            };
            // the weights depend on no earlier kernel: the first stages' W is on its way before this kernel may read x
            const int first = k_tiles < a.stages ? k_tiles : a.stages;
            const int tile0 = blockIdx.x;
            if (tile0 < n_tiles)
                for (int i = 0; i < first; ++i) load_w(i, i, tile0 * kTileCols);
            pdl_wait();
            if (tile0 < n_tiles)
                for (int i = 0; i < first; ++i) load_x(i, i);
            uint32_t it = 0;
            bool ok = true;
            for (int tile = tile0; tile < n_tiles && ok; tile += gridDim.x) {
                for (int kt = 0; kt < k_tiles; ++kt, ++it) {
                    if (tile == tile0 && kt < first) continue;           // asked for above
                    const int s = it % a.stages;
                    if (!mbar_wait(empty0 + 8 * s, ((it / a.stages) & 1) ^ 1, abort_flag)) { ok = false; break; }
                    load_w(s, kt, tile * kTileCols);
                    load_x(s, kt);
                }
            }
            if (!ok) { *abort_flag = 1; atomicMax(&g_stream_error, 2u); }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer
        const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
        const uint64_t desc0 = umma_desc(smem_addr(smem));
        const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(a.n_pad >> 3) << 17) | ((uint32_t)(kRows >> 4) << 24);
        uint32_t it = 0;
        int j = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++j) {
            const int acc = j & 1;
            ok = mbar_wait(acc_empty0 + 8 * acc, ((j >> 1) & 1) ^ 1, abort_flag);
            const uint32_t tmem_d = tmem_u + acc * 128;
            for (int kt = 0; kt < k_tiles && ok; ++kt, ++it) {
                const int s = it % a.stages;
                if (!mbar_wait(full0 + 8 * s, (it / a.stages) & 1, abort_flag)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t w_desc = desc0 + (uint64_t)((uint32_t)(s * stage_bytes) >> 4);
                const uint64_t x_desc = w_desc + (uint64_t)(kWBytes >> 4);
                if (elect_one()) {
#pragma unroll
                    for (int k = 0; k < kBK / 16; ++k)
                        umma_bf16(tmem_d, w_desc + (uint64_t)(k * 2), x_desc + (uint64_t)(k * 2), idesc, (kt > 0 || k > 0) ? 1u : 0u);
                    umma_commit(empty0 + 8 * s);
                    if (kt == k_tiles - 1) umma_commit(acc_full0 + 8 * acc);
                }
                __syncwarp();
            }
        }
        if (!ok && lane == 0) { *abort_flag = 1; atomicMax(&g_stream_error, 3u); }
    } else {
        // ---------------- epilogue: this thread holds weight row `row` of the tile, one token per column
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        int j = 0;
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++j) {
            const int acc = j & 1;
            const int n0 = tile * kTileCols;
            if (!mbar_wait(acc_full0 + 8 * acc, (j >> 1) & 1, abort_flag)) {
                if (lane == 0) { *abort_flag = 1; atomicMax(&g_stream_error, 4u); }
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (tile + (int)gridDim.x >= n_tiles) pdl_trigger();                 // this block's last tile
            const uint32_t lane_base = tmem_base + acc * 128 + ((uint32_t)(quarter * 32) << 16);
            for (int c0 = 0; c0 < a.M; c0 += 32) {
                uint32_t v[32];
                tmem_ld32(lane_base + c0, v);
                if (MODE == kSwiGLU) {
                    if (quarter >= 2) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) stage_up[i * (kRows / 2) + (row - kRows / 2)] = __uint_as_float(v[i]);
                    }
                    named_barrier(1, 128);
                    if (quarter < 2 && n0 + row < a.inter) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            if (c0 + i < a.M) {
                                const float g = __uint_as_float(v[i]), u = stage_up[i * (kRows / 2) + row];
                                out[(size_t)(c0 + i) * a.inter + n0 + row] = from_float<OutT>(g / (1.0f + expf(-g)) * u);
                            }
                        }
                    }
                    named_barrier(2, 128);
                } else if (n0 + row < a.N) {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (c0 + i < a.M) out[(size_t)(c0 + i) * a.N + n0 + row] = from_float<OutT>(__uint_as_float(v[i]));
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty0 + 8 * acc);
        }
    }
    __syncwarp();
    if (*abort_flag) {
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kPersistTmem));
}

// Row-major [rows, K] bfloat16 matrix, boxes of box_rows x 64 columns, 128-byte swizzle, zero fill outside.
int make_map(CUtensorMap* map, const void* base, long long rows, int K, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return (int)cudaErrorNotSupported;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {kBK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult rc = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return rc == CUDA_SUCCESS ? 0 : PB_ERR_BAD_SIZE;
}

int sm_count() {
    static int n = [] {
        int dev = 0, v = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) v = 0;
        return v > 0 ? v : 148;
    }();
    return n;
}

int forced(const char* name) {
    const char* v = getenv(name);
    return v ? atoi(v) : 0;
}

template <int MODE, typename OutT>
int launch(const CUtensorMap& mx, const CUtensorMap& mw, void* out, StreamArgs a, int tiles, cudaStream_t stream) {
    const int k_tiles = (a.K + kBK - 1) / kBK;
    // Slices of K: as many as give every SM a block (one block per SM then, with a deep ring); with more tiles than
    // SMs no slices and two blocks per SM (rings half as deep, the receive buffer in the ring's place).
    int splits = sm_count() / tiles;
    if (splits > kMaxCluster) splits = kMaxCluster;
    if (splits > k_tiles) splits = k_tiles;
    if (splits < 1) splits = 1;
    if (forced("PULSAR_STREAM_SPLITS") > 0) splits = forced("PULSAR_STREAM_SPLITS") < k_tiles ? forced("PULSAR_STREAM_SPLITS") : k_tiles;
    if (splits > kMaxCluster) splits = kMaxCluster;
    if (splits == 1 && forced("PULSAR_STREAM_PERSISTENT") >= 0) {
        // persistent: one block per SM, a deep ring, two accumulators
        a.splits = 1;
        a.cols_per = a.M;
        const int stage_bytes1 = kWBytes + a.n_pad * kBK * 2;
        const int up_bytes = MODE == kSwiGLU ? 32 * (kRows / 2) * 4 : 0;
        int stages1 = (220 * 1024 - 1024 - 256 - up_bytes) / stage_bytes1;
        if (stages1 > kMaxStages) stages1 = kMaxStages;
        if (forced("PULSAR_STREAM_STAGES") > 0 && forced("PULSAR_STREAM_STAGES") < stages1) stages1 = forced("PULSAR_STREAM_STAGES");
        if (stages1 < 2) return PB_ERR_BAD_SIZE;
        a.stages = stages1;
        a.recv_offset = stages1 * stage_bytes1;
        a.bar_offset = (a.recv_offset + up_bytes + 15) / 16 * 16;
        const int smem1 = a.bar_offset + 256 + 1024;
        static bool configured1 = false;
        if (!configured1) {
            cudaError_t rc = cudaFuncSetAttribute(gemm_tcgen05_stream_persistent_kernel<MODE, OutT>,
                                                  cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
            if (rc != cudaSuccess) return (int)rc;
            configured1 = true;
        }
        const int grid = tiles < sm_count() ? tiles : sm_count();
        return launch_pdl(gemm_tcgen05_stream_persistent_kernel<MODE, OutT>, grid, kThreads, smem1, stream, mx, mw, (OutT*)out, a, tiles);
    }
    a.splits = splits;
    a.cols_per = (a.M + splits - 1) / splits;
    const int stage_bytes = kWBytes + a.n_pad * kBK * 2;
    const int recv_bytes = splits * a.cols_per * kRows * 4;
    const int budget = splits > 1 ? 220 * 1024 : 110 * 1024;         // one block per SM, or two
    int stages = (budget - 1024 - 256 - (splits > 1 ? recv_bytes : 0)) / stage_bytes;
    if (stages > kMaxStages) stages = kMaxStages;
    if (forced("PULSAR_STREAM_STAGES") > 0 && forced("PULSAR_STREAM_STAGES") < stages) stages = forced("PULSAR_STREAM_STAGES");
    if (stages < 2 || (splits == 1 && stages * stage_bytes < recv_bytes)) return PB_ERR_BAD_SIZE;
    a.stages = stages;
    const int ring = stages * stage_bytes;
    a.recv_offset = splits > 1 ? ring : 0;
    a.bar_offset = (splits > 1 ? ring + recv_bytes : ring);
    a.bar_offset = (a.bar_offset + 15) / 16 * 16;
    const int smem_bytes = a.bar_offset + 256 + 1024;
    static int configured = 0;
    if (configured < smem_bytes) {
        cudaError_t rc = cudaFuncSetAttribute(gemm_tcgen05_stream_kernel<MODE, OutT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (rc != cudaSuccess) return (int)rc;
        configured = 227 * 1024;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tiles * splits);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = splits;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    return (int)cudaLaunchKernelEx(&cfg, gemm_tcgen05_stream_kernel<MODE, OutT>, mx, mw, (OutT*)out, a);
}

}  // namespace

// 1 if pb_gemm_tcgen05_stream takes this problem: 1 to 128 tokens, K a multiple of 8 (TMA strides are multiples of
// 16 bytes); SwiGLU additionally needs the gate/up halves to split evenly.
PB_EXPORT int pb_gemm_tcgen05_stream_supported(int mode, int M, int N, int K) {
    if (M <= 0 || M > 128 || N <= 0 || K <= 0 || (K % 8)) return 0;
    if (mode == kSwiGLU) return (N % 2 == 0) ? 1 : 0;
    return mode == kPlain ? 1 : 0;
}

// limit > 0: the new limit of the kernel's bounded waits in clock cycles; error >= 0: the new value of the error
// word; address: receives the word's device address.  Returns 0, or -1 when a CUDA call failed.
PB_EXPORT int pb_gemm_tcgen05_stream_wait_control(long long limit, int error, void** address) {
    return wait_control(g_stream_error, limit, error, address);
}

// mode 0: out[M, N] = x W^T (out_dtype bfloat16 or float32).  mode 1: W = [gate rows; up rows], N = 2 * inter,
// out[M, inter] = silu(x Wg^T) * (x Wu^T).  x [M, K] and W [N, K] bfloat16, 16-byte aligned, M <= 128.
PB_EXPORT int pb_gemm_tcgen05_stream(int mode, int out_dtype, const void* x, const void* w, void* out, int M, int N, int K,
                                     cudaStream_t stream) {
    if (!pb_gemm_tcgen05_stream_supported(mode, M, N, K)) return PB_ERR_BAD_SIZE;
    if ((((uintptr_t)x | (uintptr_t)w) & 15) != 0) return PB_ERR_BAD_SIZE;
    if (out_dtype != PB_BF16 && out_dtype != PB_F32) return PB_ERR_BAD_DTYPE;
    StreamArgs a{};
    a.M = M;
    a.N = N;
    a.K = K;
    a.n_pad = (M + 15) / 16 * 16;
    a.inter = mode == kSwiGLU ? N / 2 : 0;
    CUtensorMap mx, mw;
    int rc = make_map(&mx, x, M, K, a.n_pad);
    if (rc != 0) return rc;
    rc = make_map(&mw, w, N, K, mode == kSwiGLU ? kRows / 2 : kRows);
    if (rc != 0) return rc;
    if (mode == kSwiGLU) {
        const int tiles = (a.inter + kRows / 2 - 1) / (kRows / 2);
        if (out_dtype == PB_BF16) return launch<kSwiGLU, bf16>(mx, mw, out, a, tiles, stream);
        return launch<kSwiGLU, float>(mx, mw, out, a, tiles, stream);
    }
    const int tiles = (N + kRows - 1) / kRows;
    if (out_dtype == PB_BF16) return launch<kPlain, bf16>(mx, mw, out, a, tiles, stream);
    return launch<kPlain, float>(mx, mw, out, a, tiles, stream);
}
