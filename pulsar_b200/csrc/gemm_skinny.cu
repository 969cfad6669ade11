// out[M, N] = x[M, K] * W[N, K]^T for a handful of tokens (M <= 16) in bfloat16: the
// projections of a decode step, where every weight is read once and the time is the time
// to stream W from HBM.
//
// The weights take the role of the MMA's 16-row operand and the tokens that of its 8-wide
// one (mma.m16n8k16, float32 accumulators).  Weights go from global memory into registers (only
// the two k-blocks per warp that are asked for before the kernel may start pass through shared
// memory, see skinny_wide_body): a thread
// loads 32 contiguous bytes of a weight row (16 where K is no multiple of 64) straight into the
// registers of A fragments and as many bytes of a token's activations into B fragments; because a dot product does
// not care about the order of its terms, the k-index that a fragment slot stands for is
// permuted the same way on both sides, which makes the vector loads legal.  A block owns
// 16 weight rows; its 8 warps split K, keep 8 vector loads each in flight, and their
// partial sums are added in warp order through shared memory.  The 32-byte loads mark their
// lines as the first to leave L2 (weights are read once and are far larger than L2).
//
// Epilogues: plain (bfloat16 or float32 output), or SwiGLU: the block's 16 rows are 8 gate
// rows and the 8 up rows that belong to them, and it writes silu(gate) * up (float32
// gating, one rounding), so the [M, 2I] intermediate never exists.
//
// The reference calls at::linear three times for q/k/v, once for o, twice for gate/up and
// once for down, plus two elementwise kernels for the gating
// (pulsar-core/src/model/qwen3.cpp:82-84, 114, 117-119).
#include "mma_common.cuh"

#include <cstdlib>

namespace {

using namespace pb;

constexpr int kWarps = 8;
constexpr int kRows = 16;
constexpr int kBlockK = 32;      // k per two MMAs: 4 threads x 8 contiguous elements

__device__ __forceinline__ uint4 load_stream(const void* p) {      // weights: read once, keep them out of L1
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

enum { kPlain = 0, kSwiGLU = 1 };

// NT: n-tiles of 8 tokens.  Mode kSwiGLU: rows r of the block are gate rows 8*b + r (r < 8) and up rows
// inter + 8*b + (r - 8); the output has `inter` columns.
template <int NT, int MODE, typename OutT, int kUnroll>
__global__ void __launch_bounds__(kWarps * 32)
gemm_skinny_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, OutT* __restrict__ out, int M, int N, int K,
                   int inter) {
    __shared__ float red[kWarps][kRows][8 * NT + 1];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    int row_a, row_b;                                   // weight rows behind fragment rows g and g + 8
    if (MODE == kSwiGLU) { row_a = blockIdx.x * 8 + g; row_b = inter + blockIdx.x * 8 + g; }
    else { row_a = blockIdx.x * kRows + g; row_b = row_a + 8; }
    const bf16* wa_p = w + (size_t)row_a * K + 8 * t;
    const bf16* wb_p = w + (size_t)row_b * K + 8 * t;
    const bf16* x_p[NT];
    bool x_ok[NT];
#pragma unroll
    for (int n = 0; n < NT; ++n) {
        x_ok[n] = n * 8 + g < M;
        x_p[n] = x + (size_t)(x_ok[n] ? n * 8 + g : 0) * K + 8 * t;
    }
    float c[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) { c[n][0] = c[n][1] = c[n][2] = c[n][3] = 0.0f; }

    const int blocks = K / kBlockK;
    const int kb_begin = (int)((long long)blocks * warp / kWarps), kb_end = (int)((long long)blocks * (warp + 1) / kWarps);
    int kb = kb_begin;
    // The weights depend on no earlier kernel: the first batch of loads is issued before this kernel
    // waits for the one that produces x (it may have been brought onto the SM while that one finishes).
    uint4 wa[kUnroll], wb[kUnroll];
    const bool first = kb + kUnroll <= kb_end;
    if (first) {
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            wa[u] = load_stream(wa_p + (size_t)(kb + u) * kBlockK);
            wb[u] = load_stream(wb_p + (size_t)(kb + u) * kBlockK);
        }
    }
    pdl_wait();
    for (bool loaded = first; kb + kUnroll <= kb_end; kb += kUnroll, loaded = false) {
        uint4 xv[kUnroll][NT];
        if (!loaded) {
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                wa[u] = load_stream(wa_p + (size_t)(kb + u) * kBlockK);
                wb[u] = load_stream(wb_p + (size_t)(kb + u) * kBlockK);
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
#pragma unroll
            for (int n = 0; n < NT; ++n)
                xv[u][n] = x_ok[n] ? __ldg(reinterpret_cast<const uint4*>(x_p[n] + (size_t)(kb + u) * kBlockK)) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const uint32_t a1[4] = {wa[u].x, wb[u].x, wa[u].y, wb[u].y};
            const uint32_t a2[4] = {wa[u].z, wb[u].z, wa[u].w, wb[u].w};
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                mma_bf16(c[n], a1, xv[u][n].x, xv[u][n].y);
                mma_bf16(c[n], a2, xv[u][n].z, xv[u][n].w);
            }
        }
    }
    for (; kb < kb_end; ++kb) {
        const uint4 wa = load_stream(wa_p + (size_t)kb * kBlockK), wb = load_stream(wb_p + (size_t)kb * kBlockK);
        const uint32_t a1[4] = {wa.x, wb.x, wa.y, wb.y};
        const uint32_t a2[4] = {wa.z, wb.z, wa.w, wb.w};
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            const uint4 xv = x_ok[n] ? __ldg(reinterpret_cast<const uint4*>(x_p[n] + (size_t)kb * kBlockK)) : make_uint4(0, 0, 0, 0);
            mma_bf16(c[n], a1, xv.x, xv.y);
            mma_bf16(c[n], a2, xv.z, xv.w);
        }
    }
    pdl_trigger();
    // accumulator (row g | g+8, token n*8 + 2t | +1) -> shared memory, then the warps are added in order
#pragma unroll
    for (int n = 0; n < NT; ++n) {
        red[warp][g][n * 8 + 2 * t] = c[n][0];
        red[warp][g][n * 8 + 2 * t + 1] = c[n][1];
        red[warp][g + 8][n * 8 + 2 * t] = c[n][2];
        red[warp][g + 8][n * 8 + 2 * t + 1] = c[n][3];
    }
    __syncthreads();
    if (MODE == kSwiGLU) {
        for (int i = tid; i < 8 * M; i += kWarps * 32) {
            const int token = i / 8, r = i % 8;
            float gate = 0.0f, up = 0.0f;
#pragma unroll
            for (int wi = 0; wi < kWarps; ++wi) { gate += red[wi][r][token]; up += red[wi][r + 8][token]; }
            out[(size_t)token * inter + blockIdx.x * 8 + r] = from_float<OutT>(gate / (1.0f + expf(-gate)) * up);
        }
    } else {
        for (int i = tid; i < kRows * M; i += kWarps * 32) {
            const int token = i / kRows, r = i % kRows;
            float acc = 0.0f;
#pragma unroll
            for (int wi = 0; wi < kWarps; ++wi) acc += red[wi][r][token];
            out[(size_t)token * N + blockIdx.x * kRows + r] = from_float<OutT>(acc);
        }
    }
}

// The same product with 32-byte loads (ld.global.v8): a thread fetches 16 contiguous elements of a weight row,
// so a warp's request covers whole 128-byte lines of eight rows, and feeds four MMAs from one load.  K must be a
// multiple of 64.  kUnroll counts these double-width loads.
struct Wide { uint4 lo, hi; };

// kEvictFirst: the line is marked as the first to leave L2 (and L2 fetches 256 bytes at a time): weights are read
// once per step and are far larger than L2, so they should not push out what the step reads again.
template <bool kEvictFirst>
__device__ __forceinline__ Wide load_stream32(const void* p) {
    Wide v;
    if (kEvictFirst)
        asm volatile("ld.global.nc.L1::no_allocate.L2::evict_first.L2::256B.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n"
                     : "=r"(v.lo.x), "=r"(v.lo.y), "=r"(v.lo.z), "=r"(v.lo.w), "=r"(v.hi.x), "=r"(v.hi.y), "=r"(v.hi.z), "=r"(v.hi.w)
                     : "l"(p));
    else
        asm volatile("ld.global.nc.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n"
                     : "=r"(v.lo.x), "=r"(v.lo.y), "=r"(v.lo.z), "=r"(v.lo.w), "=r"(v.hi.x), "=r"(v.hi.y), "=r"(v.hi.z), "=r"(v.hi.w)
                     : "l"(p));
    return v;
}
__device__ __forceinline__ Wide load_x32(const void* p, bool ok) {
    Wide v;
    if (ok) {
        // (one 32-byte load per lane instead of two of 16 was no faster: 4.86 against 4.83 ms per step of 16 sequences)
        v.lo = __ldg(reinterpret_cast<const uint4*>(p));
        v.hi = __ldg(reinterpret_cast<const uint4*>(p) + 1);
    } else {
        v.lo = v.hi = make_uint4(0, 0, 0, 0);
    }
    return v;
}

// kPre > 0 (up to 8 tokens only: with 9 to 16 the buffer takes from the L1 cache what the tokens, which every block
// of an SM reads whole, need there; measured 5.08 against 4.83 ms per step of 16 sequences): besides the first batch
// of register loads, every warp asks for its next kPre k-blocks by cp.async into
// shared memory before the kernel waits for its predecessor, so that twice the bytes are on their way while the
// kernel before this one ends; a warp copies and reads only its own part (no block barrier), rows padded by 16
// bytes against bank conflicts.  The sums keep their order.
//
// Two fused forms take the RMSNorm between two projections, and the residual addition before it, into the
// projections themselves (a decode step then has no norm kernel between its products):
//   kAcc     float32 output that is ADDED to what ``out`` holds (the residual stream; the projection's result never
//            exists in bfloat16).  With ``fuse.next_w`` the block also prepares the norm that follows for its 16
//            columns: y = bfloat16(x_new * next_w) and the block's part of sum_k x_new[token, k]^2.
//   kScaled  the tokens come as such a prepared y; the sums of token m are scaled by rsqrt(sum / K + eps), the sum
//            being the parts added in block order within a lane, then a fixed tree (float32: the same bits every
//            time).  A block of its own (block 0 of a grid with one block more than tiles) adds them and leaves
//            each sum behind the parts in one word with a tag that says it is there; the blocks of the product
//            look for them when they start (all but the first round find them) and, if need be, once more at
//            their end, where the sums are wanted; if block 0 should not have come that far they add the parts
//            themselves in the same order.  No block waits for another.
// rmsnorm(x) W^T = rsqrt(mean(x^2) + eps) * ((x * norm_w) W^T): the per-token factor commutes with the product.

// A token's sum of squares travels as one 64-bit word, the sum beside a tag that says it is there (1): written and
// read with one scalar access each, so that whoever reads the tag 1 holds the sum that was written with it.
__device__ __forceinline__ unsigned long long pack_sum(float sum, unsigned int tag) {
    return ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(sum);
}

// rsqrt(mean(x^2) + eps) of every token into scale_s from the parts of its sum of squares; the sums themselves, tagged,
// to pairs_out where that is not null.  All warps of the block.
__device__ __forceinline__ void add_parts(const float* parts, int n_parts, int M, int K, float eps, int warp, int lane,
                                          float* scale_s, unsigned long long* pairs_out, unsigned int tag) {
    for (int token = warp; token < M; token += kWarps) {
        float sum = 0.0f;
        for (int b = lane; b < n_parts; b += 32) sum += __ldcg(parts + (size_t)b * M + token);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (lane == 0) {
            scale_s[token] = rsqrtf(sum / (float)K + eps);
            if (pairs_out != nullptr) __stcg(pairs_out + token, pack_sum(sum, tag));
        }
    }
}

struct SkinnyFuse {
    const float* next_w;      // kAcc: weight of the norm that follows, or null
    bf16* y;                  // kAcc: [M, N] prepared operand
    float* parts;             // [n_parts, M] each producing block's part of the sums of squares, then [M] 64-bit words:
                              // a token's sum and the tag that says it is there
    int n_parts;              // blocks of the producing product
    int publish;              // kScaled: block 0 leaves the sums for the others (0: every block adds the parts itself)
    float eps;
};

template <int NT, int MODE, typename OutT, int kUnroll, bool kEvictFirst, int kPre, bool kScaled = false, bool kAcc = false>
__device__ __forceinline__ void
skinny_wide_body(const bf16* __restrict__ x, const bf16* __restrict__ w, OutT* __restrict__ out, int M, int N, int K,
                 int inter, const SkinnyFuse fuse = SkinnyFuse{}) {
    constexpr int kWideK = 64;                        // k per load: 4 threads x 16 contiguous elements
    constexpr int kPreRow = kPre * 128 + 16;          // bytes of a row's prefetched part in shared memory
    __shared__ float red[kWarps][kRows][8 * NT + 1];
    __shared__ float scale_s[kScaled ? 8 * NT : 1];                 // kScaled: rsqrt(mean(x^2) + eps) per token
    __shared__ float square_s[kAcc ? 8 * NT : 1][kAcc ? kRows : 1]; // kAcc: x_new^2 of the block's columns
    __shared__ __align__(16) unsigned char pre[kPre > 0 ? kWarps : 1][kPre > 0 ? kRows : 1][kPre > 0 ? kPreRow : 16];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    // kScaled: the grid has one block more than the product has tiles.  Block 0 only adds the parts of the sums of
    // squares, leaves the sums behind them with the word that says so, and ends; it is the first block to be placed and
    // is done long before any other block reaches its end, where the sums are wanted.
    const int bid = kScaled ? (int)blockIdx.x - 1 : (int)blockIdx.x;
    if constexpr (kScaled) {
        if (bid < 0) {
            pdl_wait();
            add_parts(fuse.parts, fuse.n_parts, M, K, fuse.eps, warp, lane, scale_s,
                      reinterpret_cast<unsigned long long*>(fuse.parts + (size_t)fuse.n_parts * M), fuse.publish ? 1u : 0u);
            return;
        }
    }
    int row_a, row_b;
    if (MODE == kSwiGLU) { row_a = bid * 8 + g; row_b = inter + bid * 8 + g; }
    else { row_a = bid * kRows + g; row_b = row_a + 8; }
    const bf16* wa_p = w + (size_t)row_a * K + 16 * t;
    const bf16* wb_p = w + (size_t)row_b * K + 16 * t;
    const bf16* x_p[NT];
    bool x_ok[NT];
#pragma unroll
    for (int n = 0; n < NT; ++n) {
        x_ok[n] = n * 8 + g < M;
        x_p[n] = x + (size_t)(x_ok[n] ? n * 8 + g : 0) * K + 16 * t;
    }
    float c[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) { c[n][0] = c[n][1] = c[n][2] = c[n][3] = 0.0f; }

    const int blocks = K / kWideK;
    const int kb_begin = (int)((long long)blocks * warp / kWarps), kb_end = (int)((long long)blocks * (warp + 1) / kWarps);
    int kb = kb_begin;
    Wide wa[kUnroll], wb[kUnroll];
    const bool first = kb + kUnroll <= kb_end;
    if (first) {
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            wa[u] = load_stream32<kEvictFirst>(wa_p + (size_t)(kb + u) * kWideK);
            wb[u] = load_stream32<kEvictFirst>(wb_p + (size_t)(kb + u) * kWideK);
        }
    }
    const bool pre_ok = kPre > 0 && first && kb + kUnroll + kPre <= kb_end;      // the same for a whole warp
    if constexpr (kPre > 0) if (pre_ok) {
        // 16 rows x kPre * 128 bytes, 16 bytes per lane and copy: one copy instruction covers whole rows' parts
        constexpr int kChunks = kPre > 0 ? kPre * 8 : 1;      // 16-byte chunks of a row's part
        constexpr int kRowsPerCopy = 32 / kChunks;
        static_assert(kPre == 0 || (32 % kChunks == 0 && kRows % kRowsPerCopy == 0), "prefetch shape");
        const uint64_t policy = l2_policy_evict_first();
        const int chunk = lane % kChunks, r0 = lane / kChunks;
#pragma unroll
        for (int i = 0; i < kRows / kRowsPerCopy; ++i) {
            const int r = i * kRowsPerCopy + r0;
            int wrow;
            if (MODE == kSwiGLU) wrow = r < 8 ? bid * 8 + r : inter + bid * 8 + (r - 8);
            else wrow = bid * kRows + r;
            const bf16* src = w + (size_t)wrow * K + (size_t)(kb + kUnroll) * kWideK + chunk * 8;
            cp_async16_policy(smem_u32(&pre[warp][r][chunk * 16]), src, true, policy);
        }
        cp_async_commit();
    }
    pdl_wait();
    // What the epilogue needs from the kernel before this one is asked for now and used at the end, so that no warp
    // waits for it: the parts of the sums of squares (copied to shared memory), the residual's old value.
    float old_value = 0.0f, next_weight = 0.0f;
    unsigned long long early = 0ull;
    if constexpr (kScaled) {
        // a block that starts after block 0 is done (every block but those of the first round) finds the sums already
        if (tid < M) early = __ldcg(reinterpret_cast<const unsigned long long*>(fuse.parts + (size_t)fuse.n_parts * M) + tid);
    }
    if constexpr (kAcc) {
        // the tags that say "the sum is there" are taken back before the product behind the norm can look at them
        if (fuse.next_w != nullptr && bid == 0 && tid < M)
            __stcg(reinterpret_cast<unsigned long long*>(fuse.parts + (size_t)gridDim.x * M) + tid, 0ull);
        if (tid < kRows * M) {
            const int col = bid * kRows + tid % kRows;
            old_value = to_float(out[(size_t)(tid / kRows) * N + col]);
            if (fuse.next_w != nullptr) next_weight = __ldg(fuse.next_w + col);
        }
    }
    auto multiply = [&](const Wide& a, const Wide& b, size_t kb_at) {
        const uint32_t a1[4] = {a.lo.x, b.lo.x, a.lo.y, b.lo.y};
        const uint32_t a2[4] = {a.lo.z, b.lo.z, a.lo.w, b.lo.w};
        const uint32_t a3[4] = {a.hi.x, b.hi.x, a.hi.y, b.hi.y};
        const uint32_t a4[4] = {a.hi.z, b.hi.z, a.hi.w, b.hi.w};
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            const Wide xv = load_x32(x_p[n] + kb_at * kWideK, x_ok[n]);
            mma_bf16(c[n], a1, xv.lo.x, xv.lo.y);
            mma_bf16(c[n], a2, xv.lo.z, xv.lo.w);
            mma_bf16(c[n], a3, xv.hi.x, xv.hi.y);
            mma_bf16(c[n], a4, xv.hi.z, xv.hi.w);
        }
    };
    bool loaded = first;
    if constexpr (kPre > 0) if (pre_ok) {
        // the register batch, then (with the next register batch already asked for) the part in shared memory
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) multiply(wa[u], wb[u], (size_t)(kb + u));
        kb += kUnroll;
        loaded = kb + kPre + kUnroll <= kb_end;
        if (loaded) {
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                wa[u] = load_stream32<kEvictFirst>(wa_p + (size_t)(kb + kPre + u) * kWideK);
                wb[u] = load_stream32<kEvictFirst>(wb_p + (size_t)(kb + kPre + u) * kWideK);
            }
        }
        cp_async_wait<0>();
        __syncwarp();
#pragma unroll
        for (int j = 0; j < kPre; ++j) {
            Wide a, b;
            const unsigned char* pa = &pre[warp][g][j * 128 + t * 32];
            const unsigned char* pb = &pre[warp][g + 8][j * 128 + t * 32];
            a.lo = *reinterpret_cast<const uint4*>(pa);
            a.hi = *reinterpret_cast<const uint4*>(pa + 16);
            b.lo = *reinterpret_cast<const uint4*>(pb);
            b.hi = *reinterpret_cast<const uint4*>(pb + 16);
            multiply(a, b, (size_t)(kb + j));
        }
        kb += kPre;
    }
    // (Asking for a register pair again as soon as its k-block is multiplied, so that the next batch is on its way
    // while this one is used, was slower: 5.05 against 4.83 ms per step of 16 sequences, 3.72 against 3.66 of 8.)
    for (; kb + kUnroll <= kb_end; kb += kUnroll, loaded = false) {
        if (!loaded) {
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                wa[u] = load_stream32<kEvictFirst>(wa_p + (size_t)(kb + u) * kWideK);
                wb[u] = load_stream32<kEvictFirst>(wb_p + (size_t)(kb + u) * kWideK);
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) multiply(wa[u], wb[u], (size_t)(kb + u));
    }
    for (; kb < kb_end; ++kb) {
        const Wide a = load_stream32<kEvictFirst>(wa_p + (size_t)kb * kWideK), b = load_stream32<kEvictFirst>(wb_p + (size_t)kb * kWideK);
        multiply(a, b, (size_t)kb);
    }
    pdl_trigger();
#pragma unroll
    for (int n = 0; n < NT; ++n) {
        red[warp][g][n * 8 + 2 * t] = c[n][0];
        red[warp][g][n * 8 + 2 * t + 1] = c[n][1];
        red[warp][g + 8][n * 8 + 2 * t] = c[n][2];
        red[warp][g + 8][n * 8 + 2 * t + 1] = c[n][3];
    }
    if constexpr (kScaled) {
        const unsigned long long* pairs = reinterpret_cast<const unsigned long long*>(fuse.parts + (size_t)fuse.n_parts * M);
        unsigned long long pair = early;
        if (!__syncthreads_and(tid >= M || (pair >> 32) == 1ull)) {
            if (tid < M) pair = __ldcg(pairs + tid);                 // once more, now that block 0 has had the time
            if (!__syncthreads_and(tid >= M || (pair >> 32) == 1ull)) {
                add_parts(fuse.parts, fuse.n_parts, M, K, fuse.eps, warp, lane, scale_s, nullptr, 0u);
                pair = 0ull;
            }
        }
        if (tid < M && (pair >> 32) == 1ull) scale_s[tid] = rsqrtf(__uint_as_float((unsigned int)pair) / (float)K + fuse.eps);
    }
    __syncthreads();
    if (MODE == kSwiGLU) {
        for (int i = tid; i < 8 * M; i += kWarps * 32) {
            const int token = i / 8, r = i % 8;
            float gate = 0.0f, up = 0.0f;
#pragma unroll
            for (int wi = 0; wi < kWarps; ++wi) { gate += red[wi][r][token]; up += red[wi][r + 8][token]; }
            if constexpr (kScaled) { gate *= scale_s[token]; up *= scale_s[token]; }
            out[(size_t)token * inter + bid * 8 + r] = from_float<OutT>(gate / (1.0f + expf(-gate)) * up);
        }
    } else {
        static_assert(kRows * 8 * NT <= kWarps * 32, "one output per thread");
        const int token = tid / kRows, r = tid % kRows;
        if (tid < kRows * M) {
            float acc = 0.0f;
#pragma unroll
            for (int wi = 0; wi < kWarps; ++wi) acc += red[wi][r][token];
            if constexpr (kScaled) acc *= scale_s[token];
            const int col = bid * kRows + r;
            OutT* dst = out + (size_t)token * N + col;
            if constexpr (kAcc) {
                const float x_new = old_value + acc;
                *dst = from_float<OutT>(x_new);
                if (fuse.next_w != nullptr) {
                    fuse.y[(size_t)token * N + col] = __float2bfloat16_rn(x_new * next_weight);
                    square_s[token][r] = x_new * x_new;
                }
            } else {
                *dst = from_float<OutT>(acc);
            }
        }
        if constexpr (kAcc) {
            if (fuse.next_w != nullptr) {
                __syncthreads();
                if (tid < M) {
                    float sum = 0.0f;
#pragma unroll
                    for (int rr = 0; rr < kRows; ++rr) sum += square_s[tid][rr];
                    __stcg(fuse.parts + (size_t)bid * M + tid, sum);
                }
            }
        }
    }
}

template <int NT, int MODE, typename OutT, int kUnroll, bool kEvictFirst>
__global__ void __launch_bounds__(kWarps * 32, kUnroll <= 2 ? 3 : 2)
gemm_skinny_wide_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, OutT* __restrict__ out, int M, int N, int K,
                        int inter) {
    skinny_wide_body<NT, MODE, OutT, kUnroll, kEvictFirst, 0>(x, w, out, M, N, K, inter);
}

// With the prefetch through shared memory; the register count is held to what lets as many blocks share an SM as
// without it (three with two loads in flight, two with four).
template <int NT, int MODE, typename OutT, int kUnroll>
__global__ void __launch_bounds__(kWarps * 32, kUnroll <= 2 ? 3 : 2)
gemm_skinny_wide_prefetch_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, OutT* __restrict__ out, int M, int N,
                                 int K, int inter) {
    skinny_wide_body<NT, MODE, OutT, kUnroll, true, 2>(x, w, out, M, N, K, inter);
}

// The tokens come prepared (see SkinnyFuse): the norm's per-token factor is applied to the sums.
template <int NT, int MODE, int kUnroll, int kPre>
__global__ void __launch_bounds__(kWarps * 32, kUnroll <= 2 ? 3 : 2)
gemm_skinny_scaled_kernel(const bf16* __restrict__ y, const bf16* __restrict__ w, bf16* __restrict__ out, int M, int N, int K,
                          int inter, const SkinnyFuse fuse) {
    skinny_wide_body<NT, MODE, bf16, kUnroll, true, kPre, true, false>(y, w, out, M, N, K, inter, fuse);
}

// The projection's result added to the float32 residual stream in place (and the next norm prepared).
template <int NT, int kUnroll, int kPre>
__global__ void __launch_bounds__(kWarps * 32, kUnroll <= 2 ? 3 : 2)
gemm_skinny_accumulate_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, float* __restrict__ out, int M, int N,
                              int K, const SkinnyFuse fuse) {
    skinny_wide_body<NT, kPlain, float, kUnroll, true, kPre, false, true>(x, w, out, M, N, K, 0, fuse);
}

// 9 to 16 tokens, weights with many tiles (gate/up, the head): a block owns 32 weight rows, two groups of 16, and a
// warp feeds both groups' MMAs from one load of the tokens' activations.  With two n-tiles of tokens a warp loads as
// many bytes of activations (from L1) as of weights per k-block; over two row groups that is halved.  kSwiGLU: group r
// holds gate rows 16 b + 8 r .. + 7 and the up rows that belong to them.  K a multiple of 64, 32-byte aligned operands.
// Measured per step: 4.60 against 4.73 ms at 16 sequences, 4.18 against 4.26 at 12, 3.89 against 3.96 at 9; for up to
// 8 tokens (one n-tile) the same shape was no faster (3.586 against 3.572 ms at 8, 3.050 against 2.985 at 1).
constexpr int kTallGroups = 2;
template <int MODE, typename OutT>
__global__ void __launch_bounds__(kWarps * 32, 2)
gemm_skinny_tall_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, OutT* __restrict__ out, int M, int N, int K, int inter) {
    constexpr int NT = 2, kU = 2, kWideK = 64;
    __shared__ float red[kWarps][kTallGroups * kRows][8 * NT + 1];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const bf16* wa_p[kTallGroups];
    const bf16* wb_p[kTallGroups];
#pragma unroll
    for (int r = 0; r < kTallGroups; ++r) {
        int row_a, row_b;
        if (MODE == kSwiGLU) { row_a = blockIdx.x * 16 + 8 * r + g; row_b = inter + row_a; }
        else { row_a = blockIdx.x * 32 + 16 * r + g; row_b = row_a + 8; }
        wa_p[r] = w + (size_t)row_a * K + 16 * t;
        wb_p[r] = w + (size_t)row_b * K + 16 * t;
    }
    const bf16* x_p[NT];
    bool x_ok[NT];
#pragma unroll
    for (int n = 0; n < NT; ++n) {
        x_ok[n] = n * 8 + g < M;
        x_p[n] = x + (size_t)(x_ok[n] ? n * 8 + g : 0) * K + 16 * t;
    }
    float c[kTallGroups][NT][4];
#pragma unroll
    for (int r = 0; r < kTallGroups; ++r)
#pragma unroll
        for (int n = 0; n < NT; ++n) { c[r][n][0] = c[r][n][1] = c[r][n][2] = c[r][n][3] = 0.0f; }
    const int blocks = K / kWideK;
    const int kb_begin = (int)((long long)blocks * warp / kWarps), kb_end = (int)((long long)blocks * (warp + 1) / kWarps);
    int kb = kb_begin;
    Wide wa[kTallGroups][kU], wb[kTallGroups][kU];
    auto load_batch = [&](int at) {
#pragma unroll
        for (int u = 0; u < kU; ++u)
#pragma unroll
            for (int r = 0; r < kTallGroups; ++r) {
                wa[r][u] = load_stream32<true>(wa_p[r] + (size_t)(at + u) * kWideK);
                wb[r][u] = load_stream32<true>(wb_p[r] + (size_t)(at + u) * kWideK);
            }
    };
    auto multiply = [&](const Wide (&a)[kTallGroups], const Wide (&b)[kTallGroups], size_t kb_at) {
        Wide xv[NT];
#pragma unroll
        for (int n = 0; n < NT; ++n) xv[n] = load_x32(x_p[n] + kb_at * kWideK, x_ok[n]);
#pragma unroll
        for (int r = 0; r < kTallGroups; ++r) {
            const uint32_t a1[4] = {a[r].lo.x, b[r].lo.x, a[r].lo.y, b[r].lo.y};
            const uint32_t a2[4] = {a[r].lo.z, b[r].lo.z, a[r].lo.w, b[r].lo.w};
            const uint32_t a3[4] = {a[r].hi.x, b[r].hi.x, a[r].hi.y, b[r].hi.y};
            const uint32_t a4[4] = {a[r].hi.z, b[r].hi.z, a[r].hi.w, b[r].hi.w};
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                mma_bf16(c[r][n], a1, xv[n].lo.x, xv[n].lo.y);
                mma_bf16(c[r][n], a2, xv[n].lo.z, xv[n].lo.w);
                mma_bf16(c[r][n], a3, xv[n].hi.x, xv[n].hi.y);
                mma_bf16(c[r][n], a4, xv[n].hi.z, xv[n].hi.w);
            }
        }
    };
    bool loaded = kb + kU <= kb_end;
    if (loaded) load_batch(kb);                       // the weights depend on no kernel: asked for before the wait
    pdl_wait();
    for (; kb + kU <= kb_end; kb += kU, loaded = false) {
        if (!loaded) load_batch(kb);
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            const Wide a[kTallGroups] = {wa[0][u], wa[1][u]}, b[kTallGroups] = {wb[0][u], wb[1][u]};
            multiply(a, b, (size_t)(kb + u));
        }
    }
    for (; kb < kb_end; ++kb) {
        Wide a[kTallGroups], b[kTallGroups];
#pragma unroll
        for (int r = 0; r < kTallGroups; ++r) {
            a[r] = load_stream32<true>(wa_p[r] + (size_t)kb * kWideK);
            b[r] = load_stream32<true>(wb_p[r] + (size_t)kb * kWideK);
        }
        multiply(a, b, (size_t)kb);
    }
    pdl_trigger();
#pragma unroll
    for (int r = 0; r < kTallGroups; ++r)
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            red[warp][r * kRows + g][n * 8 + 2 * t] = c[r][n][0];
            red[warp][r * kRows + g][n * 8 + 2 * t + 1] = c[r][n][1];
            red[warp][r * kRows + g + 8][n * 8 + 2 * t] = c[r][n][2];
            red[warp][r * kRows + g + 8][n * 8 + 2 * t + 1] = c[r][n][3];
        }
    __syncthreads();
    if (MODE == kSwiGLU) {
        for (int i = tid; i < 16 * M; i += kWarps * 32) {
            const int token = i / 16, j = i % 16;
            const int row = (j / 8) * kRows + (j % 8);                 // the gate row; its up row lies 8 further
            float gate = 0.0f, up = 0.0f;
#pragma unroll
            for (int wi = 0; wi < kWarps; ++wi) { gate += red[wi][row][token]; up += red[wi][row + 8][token]; }
            out[(size_t)token * inter + blockIdx.x * 16 + j] = from_float<OutT>(gate / (1.0f + expf(-gate)) * up);
        }
    } else {
        for (int i = tid; i < kTallGroups * kRows * M; i += kWarps * 32) {
            const int token = i / (kTallGroups * kRows), r = i % (kTallGroups * kRows);
            float acc = 0.0f;
#pragma unroll
            for (int wi = 0; wi < kWarps; ++wi) acc += red[wi][r][token];
            out[(size_t)token * N + blockIdx.x * (kTallGroups * kRows) + r] = from_float<OutT>(acc);
        }
    }
}

// kUnroll: k-blocks whose weight loads a thread keeps in flight.  8 costs 128 registers, so that two blocks
// share an SM; 4 lets three share it.  A product whose blocks all fit two per SM takes 8; one with more blocks
// takes 4, so that it does not need a second, nearly empty round of blocks (the QKV product of the 8B sizes:
// 384 blocks on 148 SMs) and, with thousands of blocks (gate/up, lm_head), more of them are resident.
bool wide_enabled() {       // PULSAR_SKINNY_WIDE=0 keeps the 16-byte loads
    static const bool on = [] {
        const char* v = getenv("PULSAR_SKINNY_WIDE");
        return !(v && v[0] == '0' && v[1] == 0);
    }();
    return on;
}

bool evict_first_enabled() {       // PULSAR_SKINNY_EVICT_FIRST=0: weight loads without the L2 hints
    static const bool on = [] {
        const char* v = getenv("PULSAR_SKINNY_EVICT_FIRST");
        return !(v && v[0] == '0' && v[1] == 0);
    }();
    return on;
}

bool prefetch_enabled() {          // PULSAR_SKINNY_PREFETCH=0: no part of the weights through shared memory
    static const bool on = [] {
        const char* v = getenv("PULSAR_SKINNY_PREFETCH");
        return !(v && v[0] == '0' && v[1] == 0);
    }();
    return on;
}

template <int NT, int kU, bool kEvictFirst>
int launch_wide(int mode, int out_dtype, const bf16* xp, const bf16* wp, void* out, int M, int N, int K, cudaStream_t stream) {
    if (mode == kSwiGLU) {
        const int inter = N / 2;
        if (out_dtype != PB_BF16) return PB_ERR_BAD_DTYPE;
        return launch_pdl(gemm_skinny_wide_kernel<NT, kSwiGLU, bf16, kU, kEvictFirst>, inter / 8, kWarps * 32, 0, stream, xp, wp, (bf16*)out, M, N, K, inter);
    }
    if (out_dtype == PB_BF16)
        return launch_pdl(gemm_skinny_wide_kernel<NT, kPlain, bf16, kU, kEvictFirst>, N / kRows, kWarps * 32, 0, stream, xp, wp, (bf16*)out, M, N, K, 0);
    return launch_pdl(gemm_skinny_wide_kernel<NT, kPlain, float, kU, kEvictFirst>, N / kRows, kWarps * 32, 0, stream, xp, wp, (float*)out, M, N, K, 0);
}

template <int NT, int kU>
int launch_prefetch(int mode, int out_dtype, const bf16* xp, const bf16* wp, void* out, int M, int N, int K, cudaStream_t stream) {
    if (mode == kSwiGLU) {
        const int inter = N / 2;
        if (out_dtype != PB_BF16) return PB_ERR_BAD_DTYPE;
        return launch_pdl(gemm_skinny_wide_prefetch_kernel<NT, kSwiGLU, bf16, kU>, inter / 8, kWarps * 32, 0, stream, xp, wp, (bf16*)out, M, N, K, inter);
    }
    if (out_dtype == PB_BF16)
        return launch_pdl(gemm_skinny_wide_prefetch_kernel<NT, kPlain, bf16, kU>, N / kRows, kWarps * 32, 0, stream, xp, wp, (bf16*)out, M, N, K, 0);
    return launch_pdl(gemm_skinny_wide_prefetch_kernel<NT, kPlain, float, kU>, N / kRows, kWarps * 32, 0, stream, xp, wp, (float*)out, M, N, K, 0);
}

template <int NT, int kUnroll>
int launch_u(int mode, int out_dtype, const void* x, const void* w, void* out, int M, int N, int K, cudaStream_t stream) {
    const bf16* xp = (const bf16*)x;
    const bf16* wp = (const bf16*)w;
    if (K % 64 == 0 && (((uintptr_t)x | (uintptr_t)w) & 31) == 0 && wide_enabled()) {
        constexpr int kU = kUnroll / 2;                 // the same bytes in flight
        if (!evict_first_enabled()) return launch_wide<NT, kU, false>(mode, out_dtype, xp, wp, out, M, N, K, stream);
        if (NT == 1 && prefetch_enabled()) return launch_prefetch<1, kU>(mode, out_dtype, xp, wp, out, M, N, K, stream);
        return launch_wide<NT, kU, true>(mode, out_dtype, xp, wp, out, M, N, K, stream);
    }
    if (mode == kSwiGLU) {
        const int inter = N / 2;
        if (out_dtype != PB_BF16) return PB_ERR_BAD_DTYPE;
        return launch_pdl(gemm_skinny_kernel<NT, kSwiGLU, bf16, kUnroll>, inter / 8, kWarps * 32, 0, stream, xp, wp, (bf16*)out, M, N, K, inter);
    }
    if (out_dtype == PB_BF16)
        return launch_pdl(gemm_skinny_kernel<NT, kPlain, bf16, kUnroll>, N / kRows, kWarps * 32, 0, stream, xp, wp, (bf16*)out, M, N, K, 0);
    return launch_pdl(gemm_skinny_kernel<NT, kPlain, float, kUnroll>, N / kRows, kWarps * 32, 0, stream, xp, wp, (float*)out, M, N, K, 0);
}

int g_publish_sums = 1;

int sm_count() {
    static int n = [] {
        int dev = 0, v = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) v = 0;
        return v > 0 ? v : 148;
    }();
    return n;
}

bool tall_enabled() {              // PULSAR_SKINNY_TALL=0: 16 rows per block also for 9 to 16 tokens
    static const bool on = [] {
        const char* v = getenv("PULSAR_SKINNY_TALL");
        return !(v && v[0] == '0' && v[1] == 0);
    }();
    return on;
}

template <int NT>
int launch(int mode, int out_dtype, const void* x, const void* w, void* out, int M, int N, int K, cudaStream_t stream) {
    const int tiles = (mode == kSwiGLU) ? N / 2 / 8 : N / kRows;
    if (NT == 2 && tall_enabled() && wide_enabled() && evict_first_enabled() && K % 64 == 0 && (((uintptr_t)x | (uintptr_t)w) & 31) == 0 &&
        tiles % 2 == 0 && tiles / 2 > 2 * sm_count()) {
        const bf16* xp = (const bf16*)x;
        const bf16* wp = (const bf16*)w;
        if (mode == kSwiGLU) {
            if (out_dtype != PB_BF16) return PB_ERR_BAD_DTYPE;
            return launch_pdl(gemm_skinny_tall_kernel<kSwiGLU, bf16>, tiles / 2, kWarps * 32, 0, stream, xp, wp, (bf16*)out, M, N, K, N / 2);
        }
        if (out_dtype == PB_BF16)
            return launch_pdl(gemm_skinny_tall_kernel<kPlain, bf16>, tiles / 2, kWarps * 32, 0, stream, xp, wp, (bf16*)out, M, N, K, 0);
        return launch_pdl(gemm_skinny_tall_kernel<kPlain, float>, tiles / 2, kWarps * 32, 0, stream, xp, wp, (float*)out, M, N, K, 0);
    }
    if (tiles > 2 * sm_count()) return launch_u<NT, 4>(mode, out_dtype, x, w, out, M, N, K, stream);
    return launch_u<NT, 8>(mode, out_dtype, x, w, out, M, N, K, stream);
}

}  // namespace

// 1 if pb_gemm_skinny takes this problem (bfloat16 operands; else the caller uses the library product).
PB_EXPORT int pb_gemm_skinny_supported(int mode, int M, int N, int K) {
    if (M <= 0 || M > 16 || K <= 0 || K % kBlockK) return 0;
    if (mode == kSwiGLU) return (N % 16 == 0) ? 1 : 0;       // N = 2 * inter, inter % 8 == 0
    if (mode != kPlain) return 0;
    return (N % kRows == 0) ? 1 : 0;
}

// The fused forms take what the 32-byte loads take: K a multiple of 64, 32-byte aligned operands.
PB_EXPORT int pb_gemm_skinny_fused_supported(int mode, int M, int N, int K) {
    return (pb_gemm_skinny_supported(mode, M, N, K) && K % 64 == 0) ? 1 : 0;
}

// residual[M, N] (float32) += x[M, K] W[N, K]^T.  With next_w (float32 [N], the weight of the RMSNorm that follows) also
// y[M, N] = bfloat16(residual * next_w) and parts[N / 16, M] = each block's part of sum_n residual[m, n]^2; parts has
// room for (N / 16 + 2) * M floats: behind the parts pb_gemm_skinny_scaled keeps each token's sum with a tag, which this
// kernel sets to zero; for
// pb_gemm_skinny_scaled.
PB_EXPORT int pb_gemm_skinny_accumulate(const void* x, const void* w, float* residual, int M, int N, int K, const float* next_w,
                                        void* y, float* parts, cudaStream_t stream) {
    if (!pb_gemm_skinny_fused_supported(kPlain, M, N, K)) return PB_ERR_BAD_SIZE;
    if ((((uintptr_t)x | (uintptr_t)w) & 31) != 0) return PB_ERR_BAD_SIZE;
    if (next_w != nullptr && (y == nullptr || parts == nullptr)) return PB_ERR_BAD_SIZE;
    const bf16* xp = (const bf16*)x;
    const bf16* wp = (const bf16*)w;
    SkinnyFuse fuse{};
    fuse.next_w = next_w;
    fuse.y = (bf16*)y;
    fuse.parts = parts;
    fuse.n_parts = N / kRows;
    const int tiles = N / kRows;
    const bool many = tiles > 2 * sm_count();
#define PB_ACC(NT, KU, PRE) \
    return launch_pdl(gemm_skinny_accumulate_kernel<NT, KU, PRE>, tiles, kWarps * 32, 0, stream, xp, wp, residual, M, N, K, fuse)
    if (M <= 8) { if (many) PB_ACC(1, 2, 2); PB_ACC(1, 4, 2); }
    if (many) PB_ACC(2, 2, 0);
    PB_ACC(2, 4, 0);
#undef PB_ACC
}

// on = 0: block 0 of pb_gemm_skinny_scaled keeps its sums to itself, so that every other block takes the path on
// which it adds the parts itself (which otherwise only runs when block 0 is late).  For tests of that path.
PB_EXPORT int pb_gemm_skinny_publish_sums(int on) {
    g_publish_sums = on ? 1 : 0;
    return 0;
}

// out = (y W^T) * rsqrt(sum_m / K + eps) per token m, sum_m = the K / 16 parts of parts[K / 16, M] added in order:
// with y and parts from pb_gemm_skinny_accumulate this is rmsnorm(residual) W^T.  parts: (K / 16 + 2) * M floats,
// the tagged sums behind the parts are written here.  mode 0: bfloat16 [M, N]; mode 1: the
// SwiGLU form, bfloat16 [M, N / 2].
PB_EXPORT int pb_gemm_skinny_scaled(int mode, const void* y, const void* w, void* out, int M, int N, int K, float* parts,
                                    float eps, cudaStream_t stream) {
    if (!pb_gemm_skinny_fused_supported(mode, M, N, K) || parts == nullptr) return PB_ERR_BAD_SIZE;
    if ((((uintptr_t)y | (uintptr_t)w) & 31) != 0) return PB_ERR_BAD_SIZE;
    const bf16* yp = (const bf16*)y;
    const bf16* wp = (const bf16*)w;
    SkinnyFuse fuse{};
    fuse.parts = parts;
    fuse.n_parts = K / kRows;
    fuse.publish = g_publish_sums;
    fuse.eps = eps;
    const int tiles = (mode == kSwiGLU) ? N / 2 / 8 : N / kRows;
    const int inter = mode == kSwiGLU ? N / 2 : 0;
    const bool many = tiles > 2 * sm_count();
#define PB_SCALED(NT, MODE, KU, PRE) \
    return launch_pdl(gemm_skinny_scaled_kernel<NT, MODE, KU, PRE>, tiles + 1, kWarps * 32, 0, stream, yp, wp, (bf16*)out, M, N, K, inter, fuse)
    if (M <= 8) {
        if (mode == kSwiGLU) { if (many) PB_SCALED(1, kSwiGLU, 2, 2); PB_SCALED(1, kSwiGLU, 4, 2); }
        if (many) PB_SCALED(1, kPlain, 2, 2);
        PB_SCALED(1, kPlain, 4, 2);
    }
    if (mode == kSwiGLU) { if (many) PB_SCALED(2, kSwiGLU, 2, 0); PB_SCALED(2, kSwiGLU, 4, 0); }
    if (many) PB_SCALED(2, kPlain, 2, 0);
    PB_SCALED(2, kPlain, 4, 0);
#undef PB_SCALED
}

// mode 0: out[M, N] (out_dtype bfloat16 or float32).  mode 1: W = [gate rows; up rows] with N = 2 * inter,
// out[M, inter] = silu(x Wg^T) * (x Wu^T) in bfloat16.  x, W bfloat16, 16-byte aligned.
PB_EXPORT int pb_gemm_skinny(int mode, int out_dtype, const void* x, const void* w, void* out, int M, int N, int K,
                             cudaStream_t stream) {
    if (!pb_gemm_skinny_supported(mode, M, N, K)) return PB_ERR_BAD_SIZE;
    if ((((uintptr_t)x | (uintptr_t)w) & 15) != 0) return PB_ERR_BAD_SIZE;
    if (out_dtype != PB_BF16 && out_dtype != PB_F32) return PB_ERR_BAD_DTYPE;
    if (M <= 8) return launch<1>(mode, out_dtype, x, w, out, M, N, K, stream);
    return launch<2>(mode, out_dtype, x, w, out, M, N, K, stream);
}
