// Paged attention for any batch of query tokens: prompt portions and single decoded
// tokens side by side, causal, optional sliding window, grouped-query heads, any head
// size that is a multiple of 16 up to 256, float32 or bfloat16 storage.
//
// This is the exact kernel of the engine: one block per (query token, query head),
// scores, running maximum, sums and the output accumulate in float32 with expf.  The
// reduction order of a (token, head) pair depends only on that token's position (key
// tiles of 32 aligned to absolute key indices, tile i handled by warp i mod 4, warps
// combined in index order), so logits do not depend on how tokens were cut into steps
// or batched.  The float32 path of the model always runs it; the bfloat16 path uses
// it wherever no tensor-core kernel applies.
//
// Role in the reference: pulsar-core/src/kernels/paged_common.cu:21-142
// (attn_scalar_kernel, one CTA per (query token, q head), online softmax).  Unlike it,
// keys are stored rotated and are not rotated again on read, and partial results are
// combined in a fixed order instead of with atomics.
//
// Layouts: q, out [N, Hq, D]; pools [pages, Hkv, page_size, D]; block_table
// [S, table_stride] of page ids indexed by logical page (entries of pages that a window
// has released are never read); cu_q [S+1]; kv_len [S] (length after this step);
// seq_of_token [N].  Query token t of sequence s sits at position
// kv_len[s] - (cu_q[s+1]-cu_q[s]) + (t - cu_q[s]) and sees keys lo..p,
// lo = max(0, p - window + 1) when window > 0.
#include "common.cuh"

namespace {

using namespace pb;

constexpr int kWarps = 4;
constexpr int kMaxD = 256;
constexpr int kAcc = kMaxD / 32;

template <typename T> struct Vec;   // 16-byte vector of T
template <> struct Vec<float> { static constexpr int n = 4; };
template <> struct Vec<__nv_bfloat16> { static constexpr int n = 8; };

__device__ __forceinline__ void load16(const float* p, float (&f)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
__device__ __forceinline__ void load16(const __nv_bfloat16* p, float (&f)[8]) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
paged_attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                               T* __restrict__ out, const int* __restrict__ block_table, int table_stride,
                               const int* __restrict__ cu_q, const int* __restrict__ kv_len,
                               const int* __restrict__ seq_of_token, int Hq, int Hkv, int D, int page_size,
                               float scale, int window, const PoolBounds bounds) {
    extern __shared__ float smem[];
    float* q_s = smem;                         // [D] query, pre-multiplied by scale
    float* p_s = q_s + D;                      // [kWarps][32]
    float* m_s = p_s + kWarps * 32;            // [kWarps]
    float* l_s = m_s + kWarps;                 // [kWarps]
    float* acc_s = l_s + kWarps;               // [kWarps][D]

    const int t = blockIdx.x, h = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int s = seq_of_token[t];
    const int q0 = cu_q[s], q1 = cu_q[s + 1];
    const int p = kv_len[s] - (q1 - q0) + (t - q0);
    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const int g = h / (Hq / Hkv);
    const int* table = block_table + (size_t)s * table_stride;

    const T* qv = q + ((size_t)t * Hq + h) * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) q_s[i] = to_float(qv[i]) * scale;
    __syncthreads();

    float m_run = -INFINITY, l_run = 0.0f;
    float acc[kAcc];
#pragma unroll
    for (int i = 0; i < kAcc; ++i) acc[i] = 0.0f;

    const int first_tile = lo >> 5, last_tile = p >> 5;
    for (int tile = first_tile + warp; tile <= last_tile; tile += kWarps) {
        const int j = (tile << 5) + lane;
        const bool valid = j >= lo && j <= p;
        float sc = -INFINITY;
        if (valid) {
            int page = table[j / page_size];
            if (!page_ok(page, bounds)) page = 0;
            const T* kr = k_pool + (((size_t)page * Hkv + g) * page_size + j % page_size) * D;
            float dot = 0.0f;
            for (int d = 0; d < D; d += Vec<T>::n) {
                float kf[Vec<T>::n];
                load16(kr + d, kf);
#pragma unroll
                for (int e = 0; e < Vec<T>::n; ++e) dot = fmaf(q_s[d + e], kf[e], dot);
            }
            sc = dot;
        }
        const float m_new = fmaxf(m_run, warp_max(sc));      // finite: every tile in range has a valid key
        const float pv = valid ? expf(sc - m_new) : 0.0f;
        const float corr = expf(m_run - m_new);               // 0 on the first tile (m_run = -inf)
        l_run = l_run * corr + warp_sum(pv);
        m_run = m_new;
#pragma unroll
        for (int i = 0; i < kAcc; ++i) acc[i] *= corr;
        __syncwarp();
        p_s[warp * 32 + lane] = pv;
        __syncwarp();
        const int j0 = tile << 5;
        const int k_begin = (lo > j0) ? lo - j0 : 0;
        const int k_end = (p - j0 < 31) ? p - j0 : 31;
        for (int kk = k_begin; kk <= k_end; ++kk) {
            const int jj = j0 + kk;
            int page = table[jj / page_size];
            if (!page_ok(page, bounds)) page = 0;
            const T* vr = v_pool + (((size_t)page * Hkv + g) * page_size + jj % page_size) * D;
            const float pk = p_s[warp * 32 + kk];
#pragma unroll
            for (int i = 0; i < kAcc; ++i) {
                const int d = lane + 32 * i;
                if (d < D) acc[i] = fmaf(pk, to_float(vr[d]), acc[i]);
            }
        }
    }

    if (lane == 0) { m_s[warp] = m_run; l_s[warp] = l_run; }
#pragma unroll
    for (int i = 0; i < kAcc; ++i) {
        const int d = lane + 32 * i;
        if (d < D) acc_s[warp * D + d] = acc[i];
    }
    __syncthreads();
    float m_all = m_s[0];
#pragma unroll
    for (int w = 1; w < kWarps; ++w) m_all = fmaxf(m_all, m_s[w]);
    float l_all = 0.0f;
    float f[kWarps];
#pragma unroll
    for (int w = 0; w < kWarps; ++w) { f[w] = expf(m_s[w] - m_all); l_all += l_s[w] * f[w]; }
    T* ov = out + ((size_t)t * Hq + h) * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float o = 0.0f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) o += acc_s[w * D + d] * f[w];
        ov[d] = from_float<T>(o / l_all);
    }
}

}  // namespace

PB_EXPORT int pb_paged_attention_generic(int dtype, const void* q, const void* k_pool, const void* v_pool, void* out,
                                         const int* block_table, int table_stride, const int* cu_q, const int* kv_len,
                                         const int* seq_of_token, int n_tokens, int Hq, int Hkv, int D, int page_size,
                                         float scale, int window, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (D <= 0 || D % 16 || D > kMaxD || Hkv <= 0 || Hq % Hkv || page_size <= 0) return PB_ERR_BAD_SIZE;
    if (Hq > 65535) return PB_ERR_TOO_LARGE;
    const size_t smem = sizeof(float) * (D + kWarps * 32 + 2 * kWarps + (size_t)kWarps * D);
    dim3 grid(n_tokens, Hq);
    if (dtype == PB_F32)
        paged_attention_generic_kernel<float><<<grid, kWarps * 32, smem, stream>>>((const float*)q, (const float*)k_pool,
            (const float*)v_pool, (float*)out, block_table, table_stride, cu_q, kv_len, seq_of_token, Hq, Hkv, D, page_size,
            scale, window, pb::pool_bounds_now());
    else if (dtype == PB_BF16)
        paged_attention_generic_kernel<__nv_bfloat16><<<grid, kWarps * 32, smem, stream>>>((const __nv_bfloat16*)q,
            (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, (__nv_bfloat16*)out, block_table, table_stride, cu_q,
            kv_len, seq_of_token, Hq, Hkv, D, page_size, scale, window, pb::pool_bounds_now());
    else return PB_ERR_BAD_DTYPE;
    return launch_status();
}
