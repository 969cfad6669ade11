// Paged decode attention, split over the keys: every sequence of the batch brings one
// query token.  One block handles (split of the keys, kv head, sequence) for all query
// heads of that kv head's group, so a key or value row is fetched once for the group;
// the block writes an unnormalised partial (running maximum, sum, accumulator) per head
// to scratch memory and a second kernel merges the partials in split order.
//
// The grid does not depend on the context length: split i of n covers keys
// [lo + i*chunk, lo + (i+1)*chunk) with chunk = ceil(n_keys / n) rounded up to a tile,
// computed on the device from kv_len, so a captured launch stays valid as the
// sequences grow.  Splits past the end write an empty partial.
//
// Scores, softmax and accumulators are float32 (expf); any group size, any head size
// that is a multiple of 16 up to 256, float32 or bfloat16 storage, optional window.
//
// Role in the reference: pulsar-core/src/kernels/paged_attention.cu:295-412
// (paged_decode_split_kernel, paged_decode_combine_kernel; auto_splits :432-438).
#include "common.cuh"

#include <cstdlib>

namespace {

using namespace pb;

constexpr int kWarps = 4;
constexpr int kMaxD = 256;
constexpr int kAcc = kMaxD / 32;
constexpr int kGP = 4;          // query heads handled per pass over the keys

__device__ __forceinline__ void load_row16(const float* p, float (&f)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *reinterpret_cast<const float4*>(p + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
__device__ __forceinline__ void load_row16(const __nv_bfloat16* p, float (&f)[8]) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

// partial layout: [S, Hq, n_splits, D + 2] floats: acc[D], m, l
template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
decode_split_kernel(const T* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                    float* __restrict__ partial, const int* __restrict__ block_table, int table_stride,
                    const int* __restrict__ kv_len, int Hq, int Hkv, int D, int page_size, float scale, int window,
                    int n_splits, const PoolBounds bounds) {
    extern __shared__ float smem[];
    const int G = Hq / Hkv;
    float* q_s = smem;                                  // [kGP][D]
    float* p_s = q_s + kGP * D;                         // [kWarps][kGP][32]
    float* m_s = p_s + kWarps * kGP * 32;               // [kWarps][kGP]
    float* l_s = m_s + kWarps * kGP;                    // [kWarps][kGP]
    float* acc_s = l_s + kWarps * kGP;                  // [kWarps][kGP][D]

    const int split = blockIdx.x, kvh = blockIdx.y, s = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int p = kv_len[s] - 1;                        // position of the query token
    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const int n_keys = p - lo + 1;
    int chunk = (n_keys + n_splits - 1) / n_splits;
    chunk = (chunk + 31) & ~31;
    const int begin = lo + split * chunk;
    const int end = min(p + 1, begin + chunk);          // keys [begin, end)
    const int* table = block_table + (size_t)s * table_stride;
    const int stride = D + 2;

    for (int g0 = 0; g0 < G; g0 += kGP) {
        const int gn = min(kGP, G - g0);
        __syncthreads();
        for (int i = threadIdx.x; i < gn * D; i += blockDim.x) {
            const int g = i / D, d = i - g * D;
            q_s[g * D + d] = to_float(q[((size_t)s * Hq + kvh * G + g0 + g) * D + d]) * scale;
        }
        __syncthreads();

        float m_run[kGP], l_run[kGP], acc[kGP][kAcc];
#pragma unroll
        for (int g = 0; g < kGP; ++g) {
            m_run[g] = -INFINITY; l_run[g] = 0.0f;
#pragma unroll
            for (int i = 0; i < kAcc; ++i) acc[g][i] = 0.0f;
        }

        for (int j0 = begin + warp * 32; j0 < end; j0 += kWarps * 32) {
            const int j = j0 + lane;
            const bool valid = j < end;
            float sc[kGP];
#pragma unroll
            for (int g = 0; g < kGP; ++g) sc[g] = 0.0f;
            if (valid) {
                int page = table[j / page_size];
                if (!page_ok(page, bounds)) page = 0;
                const T* kr = k_pool + (((size_t)page * Hkv + kvh) * page_size + j % page_size) * D;
                for (int d = 0; d < D; d += 8) {
                    float kf[8];
                    load_row16(kr + d, kf);
#pragma unroll
                    for (int g = 0; g < kGP; ++g) {
                        if (g < gn) {
                            const float4 qa = *reinterpret_cast<const float4*>(q_s + g * D + d);
                            const float4 qb = *reinterpret_cast<const float4*>(q_s + g * D + d + 4);
                            sc[g] = fmaf(qa.x, kf[0], sc[g]); sc[g] = fmaf(qa.y, kf[1], sc[g]);
                            sc[g] = fmaf(qa.z, kf[2], sc[g]); sc[g] = fmaf(qa.w, kf[3], sc[g]);
                            sc[g] = fmaf(qb.x, kf[4], sc[g]); sc[g] = fmaf(qb.y, kf[5], sc[g]);
                            sc[g] = fmaf(qb.z, kf[6], sc[g]); sc[g] = fmaf(qb.w, kf[7], sc[g]);
                        }
                    }
                }
            }
            __syncwarp();
#pragma unroll
            for (int g = 0; g < kGP; ++g) {
                if (g < gn) {
                    const float m_new = fmaxf(m_run[g], warp_max(valid ? sc[g] : -INFINITY));
                    const float pv = valid ? expf(sc[g] - m_new) : 0.0f;
                    const float corr = expf(m_run[g] - m_new);
                    l_run[g] = l_run[g] * corr + warp_sum(pv);
                    m_run[g] = m_new;
#pragma unroll
                    for (int i = 0; i < kAcc; ++i) acc[g][i] *= corr;
                    p_s[(warp * kGP + g) * 32 + lane] = pv;
                }
            }
            __syncwarp();
            const int n_here = min(32, end - j0);
            for (int kk = 0; kk < n_here; ++kk) {
                const int jj = j0 + kk;
                int page = table[jj / page_size];
                if (!page_ok(page, bounds)) page = 0;
                const T* vr = v_pool + (((size_t)page * Hkv + kvh) * page_size + jj % page_size) * D;
                float vf[kAcc];
#pragma unroll
                for (int i = 0; i < kAcc; ++i) {
                    const int d = lane + 32 * i;
                    vf[i] = d < D ? to_float(vr[d]) : 0.0f;
                }
#pragma unroll
                for (int g = 0; g < kGP; ++g) {
                    if (g < gn) {
                        const float pk = p_s[(warp * kGP + g) * 32 + kk];
#pragma unroll
                        for (int i = 0; i < kAcc; ++i) acc[g][i] = fmaf(pk, vf[i], acc[g][i]);
                    }
                }
            }
        }

        // merge the warps in index order
#pragma unroll
        for (int g = 0; g < kGP; ++g) {
            if (g < gn) {
                if (lane == 0) { m_s[warp * kGP + g] = m_run[g]; l_s[warp * kGP + g] = l_run[g]; }
#pragma unroll
                for (int i = 0; i < kAcc; ++i) {
                    const int d = lane + 32 * i;
                    if (d < D) acc_s[(warp * kGP + g) * D + d] = acc[g][i];
                }
            }
        }
        __syncthreads();
        for (int i = threadIdx.x; i < gn * D; i += blockDim.x) {
            const int g = i / D, d = i - g * D;
            float m_all = -INFINITY;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) m_all = fmaxf(m_all, m_s[w * kGP + g]);
            float o = 0.0f, l_all = 0.0f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                const float f = (m_all == -INFINITY) ? 0.0f : expf(m_s[w * kGP + g] - m_all);
                o += acc_s[(w * kGP + g) * D + d] * f;
                l_all += l_s[w * kGP + g] * f;
            }
            float* dst = partial + (((size_t)s * Hq + kvh * G + g0 + g) * n_splits + split) * stride;
            dst[d] = o;
            if (d == 0) { dst[D] = m_all; dst[D + 1] = l_all; }
        }
    }
}

// One block per (sequence, head): the weights exp(m_i - m_all) of the splits are computed
// once, then every thread adds its column over the splits in split order.
template <typename T>
__global__ void decode_combine_kernel(const float* __restrict__ partial, T* __restrict__ out, int D, int n_splits) {
    __shared__ float w_s[64];                            // n_splits <= 64 (checked by the launchers)
    __shared__ float l_s;
    pdl_trigger();
    pdl_wait();
    const size_t row = blockIdx.x;                       // s * Hq + h
    const int stride = D + 2;
    const float* base = partial + row * n_splits * stride;
    // A thread's column of the first 32 splits is asked for before anything else, so that these loads, the maxima and
    // the sums are all on their way together: one trip to L2 instead of one for the weights and one per eight splits
    // (2.918 against 2.955 ms per step of one sequence with 16 splits, 3.562 against 3.578 of eight with 4).
    constexpr int kAhead = 32;
    const int d_first = threadIdx.x;
    float ahead[kAhead];
#pragma unroll
    for (int j = 0; j < kAhead; ++j) ahead[j] = (j < n_splits && d_first < D) ? __ldcg(base + j * stride + d_first) : 0.0f;
    if (threadIdx.x < 32) {
        // a lane's splits (i and i + 32): maximum and sum fetched together, so that the loads are in flight at once
        const int i0 = threadIdx.x, i1 = threadIdx.x + 32;
        const bool ok0 = i0 < n_splits, ok1 = i1 < n_splits;
        const float m0 = ok0 ? base[i0 * stride + D] : -INFINITY, l0 = ok0 ? base[i0 * stride + D + 1] : 0.0f;
        const float m1 = ok1 ? base[i1 * stride + D] : -INFINITY, l1 = ok1 ? base[i1 * stride + D + 1] : 0.0f;
        const float m_all = warp_max(fmaxf(m0, m1));
        const float w0 = (m0 > -INFINITY) ? expf(m0 - m_all) : 0.0f, w1 = (m1 > -INFINITY) ? expf(m1 - m_all) : 0.0f;
        w_s[i0] = w0;                                    // beyond n_splits: 0
        w_s[i1] = w1;
        // lanes hold disjoint splits; add them in lane order for a fixed result
        float l_part = l0 * w0 + l1 * w1;
        for (int o = 16; o > 0; o >>= 1) l_part += __shfl_xor_sync(0xffffffffu, l_part, o);
        if (threadIdx.x == 0) l_s = l_part;
    }
    __syncthreads();
    const float inv = l_s > 0.0f ? 1.0f / l_s : 0.0f;     // a sequence without keys (kv_len 0): zeros, not 0 * inf
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float o = 0.0f;
        int i = 0;
        if (d == d_first) {                               // the splits that are here already, in split order
#pragma unroll
            for (int j = 0; j < kAhead; ++j) o = fmaf(ahead[j], w_s[j], o);        // beyond n_splits: 0 * 0
            i = kAhead;
        }
        for (; i < n_splits; i += 8) {                   // eight loads in flight, added in split order
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = (i + j < n_splits) ? base[(i + j) * stride + d] : 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) o = fmaf(v[j], w_s[i + j], o);
        }
        out[row * D + d] = from_float<T>(o * inv);
    }
}

size_t split_smem(int D) {
    return sizeof(float) * ((size_t)kGP * D + kWarps * kGP * 32 + 2 * kWarps * kGP + (size_t)kWarps * kGP * D);
}

}  // namespace

// Floats of scratch the split kernel writes and the combine kernel reads.
PB_EXPORT long long pb_decode_scratch_floats(int n_seqs, int Hq, int D, int n_splits) {
    return (long long)n_seqs * Hq * n_splits * (D + 2);
}

// q, out [S, Hq, D] (one query token per sequence); partial: pb_decode_scratch_floats floats.
PB_EXPORT int pb_paged_attention_decode(int dtype, const void* q, const void* k_pool, const void* v_pool, void* out,
                                        float* partial, const int* block_table, int table_stride, const int* kv_len,
                                        int n_seqs, int Hq, int Hkv, int D, int page_size, float scale, int window,
                                        int n_splits, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (D <= 0 || D % 16 || D > kMaxD || Hkv <= 0 || Hq % Hkv || page_size <= 0 || n_splits <= 0) return PB_ERR_BAD_SIZE;
    if (Hkv > 65535 || n_seqs > 65535 || n_splits > 64) return PB_ERR_TOO_LARGE;
    const size_t smem = split_smem(D);
    dim3 grid(n_splits, Hkv, n_seqs);
    if (dtype == PB_F32) {
        decode_split_kernel<float><<<grid, kWarps * 32, smem, stream>>>((const float*)q, (const float*)k_pool,
            (const float*)v_pool, partial, block_table, table_stride, kv_len, Hq, Hkv, D, page_size, scale, window, n_splits,
            pb::pool_bounds_now());
        decode_combine_kernel<float><<<n_seqs * Hq, 128, 0, stream>>>(partial, (float*)out, D, n_splits);
    } else if (dtype == PB_BF16) {
        decode_split_kernel<__nv_bfloat16><<<grid, kWarps * 32, smem, stream>>>((const __nv_bfloat16*)q,
            (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, partial, block_table, table_stride, kv_len, Hq, Hkv, D,
            page_size, scale, window, n_splits, pb::pool_bounds_now());
        decode_combine_kernel<__nv_bfloat16><<<n_seqs * Hq, 128, 0, stream>>>(partial, (__nv_bfloat16*)out, D, n_splits);
    } else {
        return PB_ERR_BAD_DTYPE;
    }
    return launch_status();
}

// ---------------------------------------------------------------------------------------
// Entry point that allocates nothing (declared in no_alloc.h; it has no counterpart in
// the reference).
//
// Who needs it: code that drives this library from a place where device memory cannot be
// allocated any more: a host that handed all device memory to one arena at start-up and
// forbids cudaMalloc afterwards, a real-time loop that may not take the allocator's lock,
// or a plugin whose owner allows launches but no allocations.  pb_paged_attention_decode
// needs scratch memory for the per-split partial results and expects the caller to bring
// it; this variant brings its own: a fixed array in the library's device image.
//
// The array is part of every CUDA context that loads the library (4 MiB per GPU, held
// until the process exits).  Host code cannot use the array's name as an address: the
// name is only a handle on the host side.  The first call on each device therefore asks
// the runtime for the array's device address, with that device current, and keeps it.
// That first call should happen before any stream capture begins, since it is a
// synchronous runtime query.
//
// All calls share the one array.  Nothing in it has to start at zero (the split kernel
// writes every partial, empty ones included, before the combine kernel reads it), and it
// keeps whatever the last call left.  Two calls that overlap on the GPU (different
// streams, or one stream per thread) race on it: run them on one stream or order them
// with events.
#include "no_alloc.h"

#include <mutex>

// The scratch itself: file scope, in the library's device image.
static __device__ __align__(256) float g_noalloc_scratch[PB_DECODE_NOALLOC_MAX_FLOATS];

namespace {

constexpr int kMaxDevices = 64;
float* g_noalloc_ptr[kMaxDevices] = {};
std::mutex g_noalloc_mutex;

// Device address of the scratch array on the current device; looked up once per device.
int noalloc_scratch(float** out) {
    int device = -1;
    cudaError_t rc = cudaGetDevice(&device);
    if (rc != cudaSuccess) return (int)rc;
    if (device < 0 || device >= kMaxDevices) return PB_ERR_TOO_LARGE;
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (g_noalloc_ptr[device] == nullptr) {
        float* ptr = nullptr;
        rc = cudaGetSymbolAddress((void**)&ptr, g_noalloc_scratch);
        if (rc != cudaSuccess) return (int)rc;
        if (ptr == nullptr) return (int)cudaErrorInvalidSymbol;
        g_noalloc_ptr[device] = ptr;
    }
    *out = g_noalloc_ptr[device];
    return 0;
}

}  // namespace

PB_EXPORT long long pb_decode_noalloc_max_floats(void) { return PB_DECODE_NOALLOC_MAX_FLOATS; }

PB_EXPORT int pb_paged_attention_decode_noalloc(int dtype, const void* q, const void* k_pool, const void* v_pool,
                                                void* out, const int* block_table, int table_stride,
                                                const int* kv_len, int n_seqs, int Hq, int Hkv, int D, int page_size,
                                                float scale, int window, int n_splits, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (D <= 0 || Hq <= 0 || n_splits <= 0) return PB_ERR_BAD_SIZE;
    const long long need = pb_decode_scratch_floats(n_seqs, Hq, D, n_splits);
    if (need > PB_DECODE_NOALLOC_MAX_FLOATS) return PB_ERR_SCRATCH_TOO_SMALL;   // see pb_decode_noalloc_max_floats()
    float* scratch = nullptr;
    const int rc = noalloc_scratch(&scratch);
    if (rc != 0) return rc;
    return pb_paged_attention_decode(dtype, q, k_pool, v_pool, out, scratch, block_table, table_stride, kv_len, n_seqs,
                                     Hq, Hkv, D, page_size, scale, window, n_splits, stream);
}

// The merge of per-split partials alone, for kernels that write partials in this file's layout.
PB_EXPORT int pb_decode_combine(int dtype, const float* partial, void* out, int rows, int D, int n_splits,
                                cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (n_splits <= 0 || n_splits > 64) return PB_ERR_TOO_LARGE;
    if (dtype == PB_F32) return launch_pdl(decode_combine_kernel<float>, rows, 128, 0, stream, partial, (float*)out, D, n_splits);
    if (dtype == PB_BF16) return launch_pdl(decode_combine_kernel<__nv_bfloat16>, rows, 128, 0, stream, partial, (__nv_bfloat16*)out, D, n_splits);
    return PB_ERR_BAD_DTYPE;
}
