// out[M, N] = x[M, K] * W[N, K]^T for 17 to 128 tokens in bfloat16: the projections of a decode step with
// dozens of sequences, where every weight is still read once and the time is the time to stream W from HBM,
// but there are too many tokens for the kernel that keeps them in MMA fragments (gemm_skinny.cu).
//
// The operands change places against gemm_tcgen05.cu: 128 rows of W are the 128-row operand of tcgen05.mma
// (the lanes of the accumulator in tensor memory), the tokens are its narrow one (16 to 128 columns).  The work
// is cut into units of (a tile of 128 weight rows, a slice of K), as many slices as make the units fill whole
// rounds of the SMs: 4096 output features are only 32 tiles, and 192 tiles on 148 SMs are 1.3 rounds.  A
// persistent grid of one block per SM walks over the units (unit u to block u mod grid) and streams its part of
// W through one ring of TMA stages without a pause: two accumulators in tensor memory take turns, so that a
// finished unit is read out while the next one's bytes arrive.  With one slice the accumulator is stored straight
// from registers.  With more, every unit writes its float32 partial sums to a workspace (they stay in L2) and
// takes a ticket of its tile; the unit that draws the tile's last ticket adds the slices in their order and stores
// the tile (no block waits for another, the order of addition is fixed).
//
// Roles in a block (192 threads): warp 0 / one thread issues the TMA loads (W with an evict-first L2 hint:
// weights are read once per step and are far larger than L2; W of the first stages is asked for before the
// kernel waits for its predecessor, x after), warp 1 / one thread issues the MMAs, warps 2-5 read the
// accumulators.  SwiGLU: a tile is 64 gate rows and the 64 up rows that belong to them (two TMA boxes), and
// silu(gate) * up is applied where the sums are complete, so the [M, 2I] intermediate never exists.
//
// Every wait on a barrier is bounded by a clock limit; a role that gives up sets the error word, lets its copies
// land, and the block frees its tensor memory and returns.  No TMA load uses cluster multicast.
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
constexpr int kTmemColumns = 256;      // two accumulators of up to 128 columns
constexpr int kMaxStages = 8;
constexpr int kMaxSlices = 16;

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

struct StreamArgs {
    int M, N, K, inter;
    int n_pad;          // tokens rounded up to a multiple of 16: columns of an accumulator, rows of an x box
    int stages;         // TMA stages of the ring
    int slices;         // slices of K per tile
    int n_tiles;        // tiles of 128 weight rows (SwiGLU: 64 gate rows and their 64 up rows)
    int up_offset;      // bytes from the ring's start to the SwiGLU staging buffer
    int bar_offset;     // bytes from the ring's start to the barriers
    float* workspace;   // slices > 1: [n_tiles * slices][M][128] float32 partial sums
    unsigned int* tickets;   // slices > 1: one per tile, zero before the launch and after it
};

__device__ __forceinline__ void named_barrier(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// Barrier of `threads` threads that returns whether `ok` held for all of them: the epilogue warps decide together
// whether a wait ran out, so that none of them goes on to a barrier that the others have left.
__device__ __forceinline__ bool named_barrier_all(int id, int threads, bool ok) {
    uint32_t all;
    asm volatile("{\n.reg .pred p, q;\nsetp.ne.u32 q, %3, 0;\nbar.red.and.pred p, %1, %2, q;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(all) : "r"(id), "r"(threads), "r"((uint32_t)ok) : "memory");
    return all != 0;
}

constexpr int kReduceCols = 16;

// Four values to consecutive addresses: one vector store where the address allows it and all four are inside.
template <typename OutT>
__device__ __forceinline__ void store4(OutT* dst, const float v[4], int valid, bool vector_ok) {
    if (valid >= 4 && vector_ok) {
        if constexpr (sizeof(OutT) == 2) {
            __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
            uint2 packed;
            packed.x = *reinterpret_cast<uint32_t*>(&lo);
            packed.y = *reinterpret_cast<uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(dst) = packed;
        } else {
            *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
        }
    } else {
        for (int i = 0; i < 4 && i < valid; ++i) dst[i] = from_float<OutT>(v[i]);
    }
}

// Sum of `slices` partial tiles [M][128 rows] float32 (slice_stride floats apart) into rows n0.. of out[M][width],
// added in the order of the slices.  128 threads.  Plain: thread = (32 row quads, 4 column groups).  SwiGLU: rows
// 0-63 are gate rows and 64-127 their up rows, thread = (16 row quads, 8 column groups), out = silu(gate) * up.
template <int MODE, typename OutT>
__device__ __forceinline__ void reduce_tile(const float* __restrict__ base, size_t slice_stride, int slices, int M, int width,
                                            int n0, int etid, OutT* __restrict__ out) {
    constexpr int kQuads = (MODE == kSwiGLU) ? 16 : 32;
    constexpr int kGroups = 128 / kQuads;
    constexpr int kVec = (MODE == kSwiGLU) ? 2 : 1;                 // float4 loads per column and slice
    constexpr int kCols = kReduceCols / kVec;
    const int quad = etid % kQuads, group = etid / kQuads;
    const int row = quad * 4;
    const int valid = width - (n0 + row);
    if (valid <= 0) return;
    const bool vector_ok = (width % 4 == 0) && (n0 % 4 == 0) &&
                           ((reinterpret_cast<uintptr_t>(out) % (4 * sizeof(OutT))) == 0);
    for (int c0 = group; c0 < M; c0 += kGroups * kCols) {
        float4 acc[kCols][kVec];
#pragma unroll
        for (int i = 0; i < kCols; ++i)
#pragma unroll
            for (int h = 0; h < kVec; ++h) acc[i][h] = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s = 0; s < slices; ++s) {
            float4 v[kCols][kVec];
#pragma unroll
            for (int i = 0; i < kCols; ++i) {
                const int c = c0 + i * kGroups;
#pragma unroll
                for (int h = 0; h < kVec; ++h)
                    v[i][h] = c < M ? __ldcg(reinterpret_cast<const float4*>(base + s * slice_stride + (size_t)c * kRows + row + h * (kRows / 2)))
                                    : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int i = 0; i < kCols; ++i)
#pragma unroll
                for (int h = 0; h < kVec; ++h) {
                    acc[i][h].x += v[i][h].x; acc[i][h].y += v[i][h].y; acc[i][h].z += v[i][h].z; acc[i][h].w += v[i][h].w;
                }
        }
#pragma unroll
        for (int i = 0; i < kCols; ++i) {
            const int c = c0 + i * kGroups;
            if (c >= M) break;
            float r[4] = {acc[i][0].x, acc[i][0].y, acc[i][0].z, acc[i][0].w};
            if (MODE == kSwiGLU) {
                const float u[4] = {acc[i][kVec - 1].x, acc[i][kVec - 1].y, acc[i][kVec - 1].z, acc[i][kVec - 1].w};
#pragma unroll
                for (int e = 0; e < 4; ++e) r[e] = r[e] / (1.0f + expf(-r[e])) * u[e];
            }
            store4<OutT>(out + (size_t)c * width + n0 + row, r, valid, vector_ok);
        }
    }
}

template <int MODE, typename OutT>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_stream_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                           OutT* __restrict__ out, const StreamArgs a) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int x_bytes = a.n_pad * kBK * 2;
    const int stage_bytes = kWBytes + x_bytes;
    float* stage_up = reinterpret_cast<float*>(smem + a.up_offset);               // SwiGLU, one slice: [32 columns][64 rows]
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + a.bar_offset);            // full[8], empty[8], acc_full[2], acc_empty[2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kMaxStages + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* last_flag = const_cast<int*>(abort_flag) + 1;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int k_tiles = (a.K + kBK - 1) / kBK;
    const int n_units = a.n_tiles * a.slices;
    constexpr int kTileCols = (MODE == kSwiGLU) ? kRows / 2 : kRows;
    const uint32_t full0 = smem_addr(bars), empty0 = smem_addr(bars + kMaxStages);
    const uint32_t acc_full0 = smem_addr(bars + 2 * kMaxStages), acc_empty0 = smem_addr(bars + 2 * kMaxStages + 2);
    // unit u = tile * slices + slice covers k-tiles [k_tiles * slice / slices, k_tiles * (slice + 1) / slices)
    auto kt_first = [&](int unit) { return (int)((long long)k_tiles * (unit % a.slices) / a.slices); };
    auto kt_last = [&](int unit) { return (int)((long long)k_tiles * (unit % a.slices + 1) / a.slices); };

    if (tid == 0) {
        for (int s = 0; s < a.stages; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(acc_full0 + 8 * i, 1); mbar_init(acc_empty0 + 8 * i, 4); }
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
            const int unit0 = blockIdx.x;
            int first = 0;
            if (unit0 < n_units) {
                const int n_kt0 = kt_last(unit0) - kt_first(unit0);
                first = n_kt0 < a.stages ? n_kt0 : a.stages;
                for (int i = 0; i < first; ++i) load_w(i, kt_first(unit0) + i, (unit0 / a.slices) * kTileCols);
            }
            pdl_wait();
            for (int i = 0; i < first; ++i) load_x(i, kt_first(unit0) + i);
            uint32_t it = 0;
            bool ok = true;
            for (int unit = unit0; unit < n_units && ok; unit += gridDim.x) {
                const int n0 = (unit / a.slices) * kTileCols;
                for (int kt = kt_first(unit); kt < kt_last(unit); ++kt, ++it) {
                    if (unit == unit0 && (int)it < first) continue;      // asked for above
                    const int s = it % a.stages;
                    if (!mbar_wait(empty0 + 8 * s, ((it / a.stages) & 1) ^ 1, abort_flag)) { ok = false; break; }
                    load_w(s, kt, n0);
                    load_x(s, kt);
                }
            }
            if (!ok) { *abort_flag = 1; atomicMax(&g_stream_error, 2u); }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: the warp walks the loop uniformly, one elected lane issues
        const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
        const uint64_t desc0 = umma_desc(smem_addr(smem));
        // float32 accumulator, bfloat16 A and B, both K-major, N >> 3, M >> 4
        const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(a.n_pad >> 3) << 17) | ((uint32_t)(kRows >> 4) << 24);
        uint32_t it = 0;
        int j = 0;
        bool ok = true;
        for (int unit = blockIdx.x; unit < n_units && ok; unit += gridDim.x, ++j) {
            const int acc = j & 1;
            ok = mbar_wait(acc_empty0 + 8 * acc, ((j >> 1) & 1) ^ 1, abort_flag);
            const uint32_t tmem_d = tmem_u + acc * 128;
            const int kt0 = kt_first(unit), kt1 = kt_last(unit);
            for (int kt = kt0; kt < kt1 && ok; ++kt, ++it) {
                const int s = it % a.stages;
                if (!mbar_wait(full0 + 8 * s, (it / a.stages) & 1, abort_flag)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t w_desc = desc0 + (uint64_t)((uint32_t)(s * stage_bytes) >> 4);
                const uint64_t x_desc = w_desc + (uint64_t)(kWBytes >> 4);
                if (elect_one()) {
#pragma unroll
                    for (int k = 0; k < kBK / 16; ++k)
                        umma_bf16(tmem_d, w_desc + (uint64_t)(k * 2), x_desc + (uint64_t)(k * 2), idesc, (kt > kt0 || k > 0) ? 1u : 0u);
                    umma_commit(empty0 + 8 * s);
                    if (kt == kt1 - 1) umma_commit(acc_full0 + 8 * acc);
                }
                __syncwarp();
            }
        }
        if (!ok && lane == 0) { *abort_flag = 1; atomicMax(&g_stream_error, 3u); }
    } else {
        // ---------------- epilogue: this thread holds weight row `row` of the tile, one token per column
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const int etid = tid - 64;                                              // 0 .. 127 among the epilogue threads
        int j = 0;
        for (int unit = blockIdx.x; unit < n_units; unit += gridDim.x, ++j) {
            const int acc = j & 1;
            const int tile = unit / a.slices;
            const int n0 = tile * kTileCols;
            if (!named_barrier_all(4, 128, mbar_wait(acc_full0 + 8 * acc, (j >> 1) & 1, abort_flag))) {
                if (lane == 0) { *abort_flag = 1; atomicMax(&g_stream_error, 4u); }
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (unit + (int)gridDim.x >= n_units) pdl_trigger();                  // this block's last unit
            const uint32_t lane_base = tmem_base + acc * 128 + ((uint32_t)(quarter * 32) << 16);
            if (a.slices > 1) {
                // partial sums of this slice -> workspace [unit][token][128 rows] (a warp's lanes are consecutive rows)
                float* part = a.workspace + (size_t)unit * a.M * kRows;
                for (int c0 = 0; c0 < a.M; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld32(lane_base + c0, v);
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (c0 + i < a.M) __stcg(part + (size_t)(c0 + i) * kRows + row, __uint_as_float(v[i]));
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty0 + 8 * acc);                // the accumulator is free again
                named_barrier(1, 128);                                           // all partial sums are written ...
                if (etid == 0) {
                    __threadfence();                                             // ... and visible before the ticket is
                    *last_flag = atomicAdd(a.tickets + tile, 1u) == (unsigned int)(a.slices - 1) ? 1 : 0;
                }
                named_barrier(2, 128);
                if (*last_flag) {
                    // the tile's last slice to finish: add the slices in their order and store the tile.  A thread
                    // owns four consecutive rows in kReduceCols columns and has all their loads in flight at once:
                    // the loads of one slice cost one trip to L2 together, not one each.
                    __threadfence();
                    const float* base = a.workspace + (size_t)tile * a.slices * a.M * kRows;
                    const size_t slice_stride = (size_t)a.M * kRows;
                    reduce_tile<MODE, OutT>(base, slice_stride, a.slices, a.M, MODE == kSwiGLU ? a.inter : a.N, n0, etid, out);
                    if (etid == 0) a.tickets[tile] = 0;                          // ready for the next launch
                }
                named_barrier(3, 128);                                           // last_flag is read by all before it is set again
                continue;
            }
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
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);      // copies that are still in flight may land
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemColumns));
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

// Slices of K for `tiles` tiles: the fewest that make the units fill their rounds of the SMs to 0.9 or better,
// never more than the k-tiles or kMaxSlices; one slice where the tiles alone make four rounds or more (the last,
// partly filled round then costs less than the partial sums would).
int choose_slices(int tiles, int k_tiles) {
    const int sms = sm_count();
    if (tiles >= 4 * sms) return 1;
    int best = 1;
    double best_fill = 0.0;
    for (int s = 1; s <= kMaxSlices && s <= k_tiles; ++s) {
        const long long units = (long long)tiles * s;
        const long long rounds = (units + sms - 1) / sms;
        const double fill = (double)units / (double)(rounds * sms);
        if (fill > best_fill + 1e-9) { best = s; best_fill = fill; }
        if (fill >= 0.9) break;
    }
    return best;
}

template <int MODE, typename OutT>
int launch(const CUtensorMap& mx, const CUtensorMap& mw, void* out, StreamArgs a, float* workspace, long long workspace_floats,
           unsigned int* tickets, int n_tickets, cudaStream_t stream) {
    const int k_tiles = (a.K + kBK - 1) / kBK;
    int slices = choose_slices(a.n_tiles, k_tiles);
    if (forced("PULSAR_STREAM_SLICES") > 0) slices = forced("PULSAR_STREAM_SLICES") < k_tiles ? forced("PULSAR_STREAM_SLICES") : k_tiles;
    if (slices > kMaxSlices) slices = kMaxSlices;
    if (slices > 1 && (workspace == nullptr || tickets == nullptr ||
                       (long long)a.n_tiles * slices * a.M * kRows > workspace_floats || a.n_tiles > n_tickets))
        slices = 1;                                                // no room for partial sums: whole tiles only
    a.slices = slices;
    a.workspace = workspace;
    a.tickets = tickets;
    const int stage_bytes = kWBytes + a.n_pad * kBK * 2;
    const int up_bytes = MODE == kSwiGLU ? 32 * (kRows / 2) * 4 : 0;
    int stages = (220 * 1024 - 1024 - 256 - up_bytes) / stage_bytes;
    if (stages > kMaxStages) stages = kMaxStages;
    if (forced("PULSAR_STREAM_STAGES") > 0 && forced("PULSAR_STREAM_STAGES") < stages) stages = forced("PULSAR_STREAM_STAGES");
    if (stages < 2) return PB_ERR_BAD_SIZE;
    a.stages = stages;
    a.up_offset = stages * stage_bytes;
    a.bar_offset = (a.up_offset + up_bytes + 15) / 16 * 16;
    const int smem_bytes = a.bar_offset + 256 + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t rc = cudaFuncSetAttribute(gemm_tcgen05_stream_kernel<MODE, OutT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (rc != cudaSuccess) return (int)rc;
        configured = true;
    }
    const long long units = (long long)a.n_tiles * slices;
    const int grid = (int)(units < sm_count() ? units : sm_count());
    return launch_pdl(gemm_tcgen05_stream_kernel<MODE, OutT>, grid, kThreads, smem_bytes, stream, mx, mw, (OutT*)out, a);
}

}  // namespace

// 1 if pb_gemm_tcgen05_stream takes this problem: 1 to 128 tokens, K a multiple of 8 (TMA strides are multiples of
// 16 bytes); SwiGLU additionally needs the gate/up halves to split evenly.
PB_EXPORT int pb_gemm_tcgen05_stream_supported(int mode, int M, int N, int K) {
    if (M <= 0 || M > 128 || N <= 0 || K <= 0 || (K % 8)) return 0;
    if (mode == kSwiGLU) return (N % 2 == 0) ? 1 : 0;
    return mode == kPlain ? 1 : 0;
}

// What the kernel wants for this problem in order to cut K into slices: `floats` of float32 workspace and
// `tickets` ticket words; both 0 when it works on whole tiles.
PB_EXPORT int pb_gemm_tcgen05_stream_workspace(int mode, int M, int N, int K, long long* floats, int* tickets) {
    const int tiles = mode == kSwiGLU ? (N / 2 + kRows / 2 - 1) / (kRows / 2) : (N + kRows - 1) / kRows;
    int slices = choose_slices(tiles, (K + kBK - 1) / kBK);
    if (forced("PULSAR_STREAM_SLICES") > 0) slices = forced("PULSAR_STREAM_SLICES");
    if (slices > kMaxSlices) slices = kMaxSlices;
    *tickets = slices > 1 ? tiles : 0;
    *floats = slices > 1 ? (long long)tiles * slices * M * kRows : 0;
    return 0;
}

// limit > 0: the new limit of the kernel's bounded waits in clock cycles; error >= 0: the new value of the error
// word; address: receives the word's device address.  Returns 0, or -1 when a CUDA call failed.
PB_EXPORT int pb_gemm_tcgen05_stream_wait_control(long long limit, int error, void** address) {
    return wait_control(g_stream_error, limit, error, address);
}

// mode 0: out[M, N] = x W^T (out_dtype bfloat16 or float32).  mode 1: W = [gate rows; up rows], N = 2 * inter,
// out[M, inter] = silu(x Wg^T) * (x Wu^T).  x [M, K] and W [N, K] bfloat16, 16-byte aligned, M <= 128.
// workspace (workspace_floats float32) and tickets (n_tickets words, zero; the kernel leaves them zero) let the
// kernel cut K into slices; without them, or where they are too small, it works on whole tiles.
PB_EXPORT int pb_gemm_tcgen05_stream(int mode, int out_dtype, const void* x, const void* w, void* out, int M, int N, int K,
                                     float* workspace, long long workspace_floats, unsigned int* tickets, int n_tickets,
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
        a.n_tiles = (a.inter + kRows / 2 - 1) / (kRows / 2);
        if (out_dtype == PB_BF16) return launch<kSwiGLU, bf16>(mx, mw, out, a, workspace, workspace_floats, tickets, n_tickets, stream);
        return launch<kSwiGLU, float>(mx, mw, out, a, workspace, workspace_floats, tickets, n_tickets, stream);
    }
    a.n_tiles = (N + kRows - 1) / kRows;
    if (out_dtype == PB_BF16) return launch<kPlain, bf16>(mx, mw, out, a, workspace, workspace_floats, tickets, n_tickets, stream);
    return launch<kPlain, float>(mx, mw, out, a, workspace, workspace_floats, tickets, n_tickets, stream);
}
