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
        v.lo = __ldg(reinterpret_cast<const uint4*>(p));
        v.hi = __ldg(reinterpret_cast<const uint4*>(p) + 1);
    } else {
        v.lo = v.hi = make_uint4(0, 0, 0, 0);
    }
    return v;
}

// kPre > 0: besides the first batch of register loads, every warp asks for its next kPre k-blocks by cp.async into
// shared memory before the kernel waits for its predecessor, so that twice the bytes are on their way while the
// kernel before this one ends; a warp copies and reads only its own part (no block barrier), rows padded by 16
// bytes against bank conflicts.  The sums keep their order.
template <int NT, int MODE, typename OutT, int kUnroll, bool kEvictFirst, int kPre>
__device__ __forceinline__ void
skinny_wide_body(const bf16* __restrict__ x, const bf16* __restrict__ w, OutT* __restrict__ out, int M, int N, int K,
                 int inter) {
    constexpr int kWideK = 64;                        // k per load: 4 threads x 16 contiguous elements
    constexpr int kPreRow = kPre * 128 + 16;          // bytes of a row's prefetched part in shared memory
    __shared__ float red[kWarps][kRows][8 * NT + 1];
    __shared__ __align__(16) unsigned char pre[kPre > 0 ? kWarps : 1][kPre > 0 ? kRows : 1][kPre > 0 ? kPreRow : 16];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    int row_a, row_b;
    if (MODE == kSwiGLU) { row_a = blockIdx.x * 8 + g; row_b = inter + blockIdx.x * 8 + g; }
    else { row_a = blockIdx.x * kRows + g; row_b = row_a + 8; }
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
            if (MODE == kSwiGLU) wrow = r < 8 ? blockIdx.x * 8 + r : inter + blockIdx.x * 8 + (r - 8);
            else wrow = blockIdx.x * kRows + r;
            const bf16* src = w + (size_t)wrow * K + (size_t)(kb + kUnroll) * kWideK + chunk * 8;
            cp_async16_policy(smem_u32(&pre[warp][r][chunk * 16]), src, true, policy);
        }
        cp_async_commit();
    }
    pdl_wait();
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

template <int NT, int MODE, typename OutT, int kUnroll, bool kEvictFirst>
__global__ void __launch_bounds__(kWarps * 32)
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

template <int kU>
int launch_prefetch(int mode, int out_dtype, const bf16* xp, const bf16* wp, void* out, int M, int N, int K, cudaStream_t stream) {
    if (mode == kSwiGLU) {
        const int inter = N / 2;
        if (out_dtype != PB_BF16) return PB_ERR_BAD_DTYPE;
        return launch_pdl(gemm_skinny_wide_prefetch_kernel<1, kSwiGLU, bf16, kU>, inter / 8, kWarps * 32, 0, stream, xp, wp, (bf16*)out, M, N, K, inter);
    }
    if (out_dtype == PB_BF16)
        return launch_pdl(gemm_skinny_wide_prefetch_kernel<1, kPlain, bf16, kU>, N / kRows, kWarps * 32, 0, stream, xp, wp, (bf16*)out, M, N, K, 0);
    return launch_pdl(gemm_skinny_wide_prefetch_kernel<1, kPlain, float, kU>, N / kRows, kWarps * 32, 0, stream, xp, wp, (float*)out, M, N, K, 0);
}

template <int NT, int kUnroll>
int launch_u(int mode, int out_dtype, const void* x, const void* w, void* out, int M, int N, int K, cudaStream_t stream) {
    const bf16* xp = (const bf16*)x;
    const bf16* wp = (const bf16*)w;
    if (K % 64 == 0 && (((uintptr_t)x | (uintptr_t)w) & 31) == 0 && wide_enabled()) {
        constexpr int kU = kUnroll / 2;                 // the same bytes in flight
        if (!evict_first_enabled()) return launch_wide<NT, kU, false>(mode, out_dtype, xp, wp, out, M, N, K, stream);
        if (NT == 1 && prefetch_enabled()) return launch_prefetch<kU>(mode, out_dtype, xp, wp, out, M, N, K, stream);
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

int sm_count() {
    static int n = [] {
        int dev = 0, v = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) v = 0;
        return v > 0 ? v : 148;
    }();
    return n;
}

template <int NT>
int launch(int mode, int out_dtype, const void* x, const void* w, void* out, int M, int N, int K, cudaStream_t stream) {
    const int tiles = (mode == kSwiGLU) ? N / 2 / 8 : N / kRows;
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
