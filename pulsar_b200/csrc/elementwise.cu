// Memory-bound kernels of the decoder step: embedding gather, residual-add + RMSNorm,
// rotary tables from explicit positions, fused per-head q/k RMSNorm + rotation +
// KV-page write, SwiGLU gating.
//
// The residual stream is float32 in both precisions; activations between kernels are
// T (float or bfloat16).  Sums of squares, rsqrt, angles, rotation and gating are
// computed in float32 (angles in float64) and rounded once on store.
//
// What the reference does with separate kernels and library calls:
//   rmsnorm        pulsar-core/src/kernels/rmsnorm.cu:17-51
//   rope           pulsar-core/src/kernels/rope.cu:27-52, rope_common.cuh:19-43
//   write_kv       pulsar-core/src/kernels/paged_attention.cu:47-70
//   q/k-norm       pulsar-core/src/model/qwen3.cpp:88-91 (two more rmsnorm launches)
//   silu(gate)*up  pulsar-core/src/model/qwen3.cpp:119 (two ATen kernels)
//   embedding      pulsar-core/src/model/paged_forward.cpp:89 (index_select)
#include "common.cuh"

namespace {

using namespace pb;

// ---------------------------------------------------------------- embedding
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids, float* __restrict__ out,
                             int width, int vocab) {
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (size_t)t * width;
    if (id < 0 || id >= vocab) {   // the host validates ids; never read out of the table
        for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = 0.0f;
        return;
    }
    const T* row = table + (size_t)id * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = to_float(row[i]);
}

// ---------------------------------------------------------------- residual add + RMSNorm
// One block per output row r.  Source row = rows ? rows[r] : r.
//   x = residual[src] (+ delta[src]);  if write_back: residual[src] = x
//   out[r] = x * rsqrt(mean(x^2) + eps) * weight
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                   const float* __restrict__ weight, T* __restrict__ out,
                                   const int* __restrict__ rows, int width, float eps, int write_back) {
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float* res = residual + (size_t)src * width;
    const T* del = delta ? delta + (size_t)src * width : nullptr;
    float local = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float x = res[i];
        if (del) x += to_float(del[i]);
        if (write_back) res[i] = x;
        local += x * x;
    }
    const float total = block_sum(local, scratch);
    const float inv = rsqrtf(total / (float)width + eps);
    T* o = out + (size_t)r * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float x = res[i];                       // own write of pass one when write_back
        if (del && !write_back) x += to_float(del[i]);
        o[i] = from_float<T>(x * inv * weight[i]);
    }
}

// ---------------------------------------------------------------- rotary tables
// cos/sin [N, half] of angle = position * quadrants_per_position[j] * pi/2.  The
// product is formed in float64 and whole quadrants are removed there (exact), so only
// a remainder below half a quadrant is rounded to float32 before sincosf.
__global__ void rope_table_kernel(const int* __restrict__ positions, const double* __restrict__ quadrants_per_position,
                                  float* __restrict__ cos_out, float* __restrict__ sin_out, int half) {
    const int t = blockIdx.x;
    const double p = (double)positions[t];
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        const double quadrants = p * quadrants_per_position[j];
        const double whole = nearbyint(quadrants);
        const float reduced = (float)(quadrants - whole) * 1.57079632679489662f;
        float s, c;
        sincosf(reduced, &s, &c);
        float co, si;
        switch ((int)((long long)whole) & 3) {
            case 0: co = c; si = s; break;
            case 1: co = -s; si = c; break;
            case 2: co = -c; si = -s; break;
            default: co = s; si = -c; break;
        }
        cos_out[(size_t)t * half + j] = co;
        sin_out[(size_t)t * half + j] = si;
    }
}

// ---------------------------------------------------------------- q/k norm + rotation + KV write
// One warp per (token, head) over the fused projection row
//   qkv[t] = [ q: Hq*D | k: Hkv*D | v: Hkv*D ].
// q heads: optional RMSNorm over D with q_weight, rotation of the first `rotary` dims
// (rotate_half pairs j, j + rotary/2), written to q_out[t, h, :].
// k heads: the same with k_weight, written into the key page of the token's slot.
// v heads: copied into the value page.  Pools are [pages, Hkv, page_size, D].
template <typename T>
__global__ void qk_norm_rope_write_kernel(const T* __restrict__ qkv, T* __restrict__ q_out,
                                          T* __restrict__ k_pool, T* __restrict__ v_pool,
                                          const int* __restrict__ slots,
                                          const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                          const float* __restrict__ q_weight, const float* __restrict__ k_weight,
                                          float eps, int Hq, int Hkv, int D, int rotary, int page_size) {
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31;
    const int head = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int heads = Hq + 2 * Hkv;
    if (head >= heads) return;
    const T* src = qkv + (size_t)t * heads * D + (size_t)head * D;
    const bool is_q = head < Hq, is_k = !is_q && head < Hq + Hkv;
    T* dst;
    if (is_q) {
        dst = q_out + ((size_t)t * Hq + head) * D;
    } else {
        const int slot = slots[t];
        if (slot < 0) return;
        const int kvh = is_k ? head - Hq : head - Hq - Hkv;
        const size_t at = (((size_t)(slot / page_size) * Hkv + kvh) * page_size + slot % page_size) * D;
        dst = (is_k ? k_pool : v_pool) + at;
    }
    if (!is_q && !is_k) {
        for (int i = lane; i < D; i += 32) dst[i] = src[i];
        return;
    }
    const float* w = is_q ? q_weight : k_weight;
    float inv = 1.0f;
    if (w) {
        float ss = 0.0f;
        for (int i = lane; i < D; i += 32) { const float x = to_float(src[i]); ss += x * x; }
        ss = warp_sum(ss);
        inv = rsqrtf(ss / (float)D + eps);
    }
    const int half = rotary >> 1;
    const float* ct = cos_t + (size_t)t * half;
    const float* st = sin_t + (size_t)t * half;
    for (int j = lane; j < half; j += 32) {
        float a = to_float(src[j]) * inv, b = to_float(src[j + half]) * inv;
        if (w) { a *= w[j]; b *= w[j + half]; }
        const float c = ct[j], s = st[j];
        dst[j] = from_float<T>(a * c - b * s);
        dst[j + half] = from_float<T>(b * c + a * s);
    }
    for (int i = rotary + lane; i < D; i += 32) {
        float a = to_float(src[i]) * inv;
        if (w) a *= w[i];
        dst[i] = from_float<T>(a);
    }
}

// ---------------------------------------------------------------- SwiGLU gating
// out[t, i] = silu(gu[t, i]) * gu[t, I + i], silu(z) = z / (1 + exp(-z)); one rounding.
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter, size_t total) {
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / inter;
        const int i = (int)(idx - t * inter);
        const float g = to_float(gu[t * 2 * inter + i]);
        const float u = to_float(gu[t * 2 * inter + inter + i]);
        out[idx] = from_float<T>(g / (1.0f + expf(-g)) * u);
    }
}

int block_for(int width) {
    int b = 32;
    while (b < 1024 && b * 4 < width) b <<= 1;
    return b;
}

}  // namespace

PB_EXPORT int pb_embed(int dtype, const void* table, const int* ids, float* out, int n, int width, int vocab,
                       cudaStream_t stream) {
    if (n <= 0) return 0;
    const int b = block_for(width);
    if (dtype == PB_F32) embed_kernel<float><<<n, b, 0, stream>>>((const float*)table, ids, out, width, vocab);
    else if (dtype == PB_BF16) embed_kernel<__nv_bfloat16><<<n, b, 0, stream>>>((const __nv_bfloat16*)table, ids, out, width, vocab);
    else return PB_ERR_BAD_DTYPE;
    return launch_status();
}

PB_EXPORT int pb_add_rmsnorm(int dtype, float* residual, const void* delta, const float* weight, void* out,
                             const int* rows, int n_out, int width, float eps, int write_back, cudaStream_t stream) {
    if (n_out <= 0) return 0;
    if (rows && write_back) return PB_ERR_BAD_SIZE;   // gathered rows are read-only
    const int b = block_for(width);
    if (dtype == PB_F32)
        add_rmsnorm_kernel<float><<<n_out, b, 0, stream>>>(residual, (const float*)delta, weight, (float*)out, rows, width, eps, write_back);
    else if (dtype == PB_BF16)
        add_rmsnorm_kernel<__nv_bfloat16><<<n_out, b, 0, stream>>>(residual, (const __nv_bfloat16*)delta, weight, (__nv_bfloat16*)out, rows, width, eps, write_back);
    else return PB_ERR_BAD_DTYPE;
    return launch_status();
}

PB_EXPORT int pb_rope_table(const int* positions, const double* quadrants_per_position, float* cos_out, float* sin_out,
                            int n, int half, cudaStream_t stream) {
    if (n <= 0 || half <= 0) return 0;
    int b = 32;
    while (b < half && b < 256) b <<= 1;
    rope_table_kernel<<<n, b, 0, stream>>>(positions, quadrants_per_position, cos_out, sin_out, half);
    return launch_status();
}

PB_EXPORT int pb_qk_norm_rope_write(int dtype, const void* qkv, void* q_out, void* k_pool, void* v_pool, const int* slots,
                                    const float* cos_t, const float* sin_t, const float* q_weight, const float* k_weight,
                                    float eps, int n, int Hq, int Hkv, int D, int rotary, int page_size,
                                    cudaStream_t stream) {
    if (n <= 0) return 0;
    if (rotary < 0 || rotary > D || (rotary & 1) || page_size <= 0) return PB_ERR_BAD_SIZE;
    const int heads = Hq + 2 * Hkv;
    const int warps = 4;
    dim3 grid(n, (heads + warps - 1) / warps);
    if (dtype == PB_F32)
        qk_norm_rope_write_kernel<float><<<grid, warps * 32, 0, stream>>>((const float*)qkv, (float*)q_out, (float*)k_pool, (float*)v_pool,
            slots, cos_t, sin_t, q_weight, k_weight, eps, Hq, Hkv, D, rotary, page_size);
    else if (dtype == PB_BF16)
        qk_norm_rope_write_kernel<__nv_bfloat16><<<grid, warps * 32, 0, stream>>>((const __nv_bfloat16*)qkv, (__nv_bfloat16*)q_out,
            (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, slots, cos_t, sin_t, q_weight, k_weight, eps, Hq, Hkv, D, rotary, page_size);
    else return PB_ERR_BAD_DTYPE;
    return launch_status();
}

PB_EXPORT int pb_silu_mul(int dtype, const void* gate_up, void* out, int n, int inter, cudaStream_t stream) {
    if (n <= 0) return 0;
    const size_t total = (size_t)n * inter;
    const int b = 256;
    size_t blocks = (total + b - 1) / b;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (dtype == PB_F32) silu_mul_kernel<float><<<(int)blocks, b, 0, stream>>>((const float*)gate_up, (float*)out, inter, total);
    else if (dtype == PB_BF16) silu_mul_kernel<__nv_bfloat16><<<(int)blocks, b, 0, stream>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter, total);
    else return PB_ERR_BAD_DTYPE;
    return launch_status();
}
