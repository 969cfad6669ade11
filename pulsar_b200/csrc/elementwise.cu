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

#include <cstdlib>
#include <cstring>

namespace pb {
bool pdl_enabled() {
    static const bool on = [] {
        const char* v = std::getenv("PULSAR_PDL");
        return !(v && std::strcmp(v, "0") == 0);
    }();
    return on;
}
}  // namespace pb

namespace {

using namespace pb;

// ---------------------------------------------------------------- embedding
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids, float* __restrict__ out,
                             int width, int vocab, float scale) {
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (size_t)t * width;
    if (id < 0 || id >= vocab) {   // the host validates ids; never read out of the table
        for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = 0.0f;
        return;
    }
    const T* row = table + (size_t)id * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = to_float(row[i]) * scale;
}

// logits *= scale, then cap * tanh(logits / cap) where cap > 0: what some architectures put behind their head.
__global__ void scale_cap_kernel(float* __restrict__ x, size_t n, float scale, float cap) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float v = x[i] * scale;
        if (cap > 0.0f) v = cap * tanhf(v / cap);
        x[i] = v;
    }
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

// The same with the row held in registers: 4 elements per thread and vector (VPT vectors
// per thread), one read of every input, vector loads and stores.  width % 4 == 0.
__device__ __forceinline__ void load4(const float* p, float (&v)[4]) {
    const float4 f = *reinterpret_cast<const float4*>(p);
    v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&v)[4]) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    v[0] = __uint_as_float(u.x << 16); v[1] = __uint_as_float(u.x & 0xffff0000u);
    v[2] = __uint_as_float(u.y << 16); v[3] = __uint_as_float(u.y & 0xffff0000u);
}
__device__ __forceinline__ void store4(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float (&v)[4]) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
}

template <typename T, int VPT>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                       const float* __restrict__ weight, T* __restrict__ out,
                                       const int* __restrict__ rows, int width, float eps, int write_back) {
    __shared__ float scratch[32];
    pdl_trigger();      // a short kernel: let the next one (a weight-streaming product) start fetching its weights now
    // the norm's weight depends on no kernel: it is here before the row is, not fetched after the sum is known
    float w[VPT][4];
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        const int i = (threadIdx.x + v * blockDim.x) * 4;
        if (i < width) load4(weight + i, w[v]);
    }
    pdl_wait();
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float* res = residual + (size_t)src * width;
    const T* del = delta ? delta + (size_t)src * width : nullptr;
    float x[VPT][4];
    float local = 0.0f;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        const int i = (threadIdx.x + v * blockDim.x) * 4;
        if (i < width) {
            load4(res + i, x[v]);
            if (del) {
                float d[4];
                load4(del + i, d);
#pragma unroll
                for (int e = 0; e < 4; ++e) x[v][e] += d[e];
            }
            if (write_back) store4(res + i, x[v]);
#pragma unroll
            for (int e = 0; e < 4; ++e) local += x[v][e] * x[v][e];
        }
    }
    const float total = block_sum(local, scratch);
    const float inv = rsqrtf(total / (float)width + eps);
    T* o = out + (size_t)r * width;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        const int i = (threadIdx.x + v * blockDim.x) * 4;
        if (i < width) {
            float y[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) y[e] = x[v][e] * inv * w[v][e];
            store4(o + i, y);
        }
    }
}

// ---------------------------------------------------------------- rotary tables
// cos/sin [N, half] of angle = position * quadrants_per_position[j] * pi/2.  The angle is kept in
// half-turns (angle / pi) in float64; whole turns are taken off there, which is exact, and what is
// left is folded into [-1/2, 1/2] half-turns (sin(pi r) = sin(pi (sign(r) - r)), the cosine changes
// sign; exact too).  Only that remainder is rounded to float32, and sincospif takes it from there,
// so the rounding of the argument never grows with the position.  (The reference reduces by whole
// quadrants and picks among four cases: pulsar-core/src/kernels/rope_common.cuh:19-43.)
__global__ void rope_table_kernel(const int* __restrict__ positions, const double* __restrict__ quadrants_per_position,
                                  float* __restrict__ cos_out, float* __restrict__ sin_out, int half) {
    const int t = blockIdx.x;
    const double p = (double)positions[t];
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        const double half_turns = p * quadrants_per_position[j] * 0.5;
        double r = half_turns - 2.0 * rint(half_turns * 0.5);          // in [-1, 1]
        const bool folded = fabs(r) > 0.5;
        if (folded) r = copysign(1.0, r) - r;
        float si, co;
        sincospif((float)r, &si, &co);
        cos_out[(size_t)t * half + j] = folded ? -co : co;
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
                                          float eps, int Hq, int Hkv, int D, int rotary, int page_size, const PoolBounds bounds) {
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
        if (slot < 0 || !slot_ok(slot, page_size, bounds)) return;
        const int kvh = is_k ? head - Hq : head - Hq - Hkv;
        const size_t at = (((size_t)(slot / page_size) * Hkv + kvh) * page_size + slot % page_size) * D;
        dst = (is_k ? k_pool : v_pool) + at;
    }
    if (!is_q && !is_k) {
        if ((D * sizeof(T)) % 16 == 0) {                   // rows are 16-byte aligned: copy vectors
            const uint4* s16 = reinterpret_cast<const uint4*>(src);
            uint4* d16 = reinterpret_cast<uint4*>(dst);
            for (int i = lane; i < (int)(D * sizeof(T) / 16); i += 32) d16[i] = s16[i];
        } else {
            for (int i = lane; i < D; i += 32) dst[i] = src[i];
        }
        return;
    }
    const float* w = is_q ? q_weight : k_weight;
    if (sizeof(T) == 2 && rotary == D && (D & 3) == 0) {
        // bfloat16, full rotation: each lane takes element pairs (2i, 2i+1) of both halves with 4-byte accesses.
        const int half = D >> 1;
        const int pairs = half >> 1;                       // pairs per half
        const uint32_t* s32 = reinterpret_cast<const uint32_t*>(src);
        uint32_t* d32 = reinterpret_cast<uint32_t*>(dst);
        float ss = 0.0f;
        for (int i = lane; i < pairs; i += 32) {
            const uint32_t a = s32[i], b = s32[i + pairs];
            const float a0 = __uint_as_float(a << 16), a1 = __uint_as_float(a & 0xffff0000u);
            const float b0 = __uint_as_float(b << 16), b1 = __uint_as_float(b & 0xffff0000u);
            ss += a0 * a0 + a1 * a1 + b0 * b0 + b1 * b1;
        }
        float inv = 1.0f;
        if (w) inv = rsqrtf(warp_sum(ss) / (float)D + eps);
        const float2* ct2 = reinterpret_cast<const float2*>(cos_t + (size_t)t * half);
        const float2* st2 = reinterpret_cast<const float2*>(sin_t + (size_t)t * half);
        for (int i = lane; i < pairs; i += 32) {
            const uint32_t a = s32[i], b = s32[i + pairs];
            float a0 = __uint_as_float(a << 16) * inv, a1 = __uint_as_float(a & 0xffff0000u) * inv;
            float b0 = __uint_as_float(b << 16) * inv, b1 = __uint_as_float(b & 0xffff0000u) * inv;
            if (w) {
                const float2 wa = reinterpret_cast<const float2*>(w)[i], wb = reinterpret_cast<const float2*>(w)[i + pairs];
                a0 *= wa.x; a1 *= wa.y; b0 *= wb.x; b1 *= wb.y;
            }
            const float2 c = ct2[i], sn = st2[i];
            const __nv_bfloat162 lo = __floats2bfloat162_rn(a0 * c.x - b0 * sn.x, a1 * c.y - b1 * sn.y);
            const __nv_bfloat162 hi = __floats2bfloat162_rn(b0 * c.x + a0 * sn.x, b1 * c.y + a1 * sn.y);
            d32[i] = *reinterpret_cast<const uint32_t*>(&lo);
            d32[i + pairs] = *reinterpret_cast<const uint32_t*>(&hi);
        }
        return;
    }
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

// The common case (bfloat16, head size 128, the whole head rotates) with more work per warp:
// a warp takes four heads of one token, issues all of its loads first, and shares the token's
// cos/sin and the norm weights between the heads.  Lane l holds elements 2l, 2l+1 of both halves.
constexpr int kRopeHeadsPerWarp = 4;
__global__ void __launch_bounds__(128)
qk_norm_rope_write_bf16_d128_kernel(const uint32_t* __restrict__ qkv, uint32_t* __restrict__ q_out,
                                    uint32_t* __restrict__ k_pool, uint32_t* __restrict__ v_pool,
                                    const int* __restrict__ slots, const float2* __restrict__ cos_t,
                                    const float2* __restrict__ sin_t, const float2* __restrict__ q_weight,
                                    const float2* __restrict__ k_weight, float eps, int Hq, int Hkv, int page_size, const PoolBounds bounds) {
    pdl_trigger();
    const int t = blockIdx.x, lane = threadIdx.x & 31;
    // the norms' weights depend on no kernel: they are here before the rows are
    float2 qw_a = make_float2(1.f, 1.f), qw_b = qw_a, kw_a = qw_a, kw_b = qw_a;
    if (q_weight) { qw_a = q_weight[lane]; qw_b = q_weight[lane + 32]; }
    if (k_weight) { kw_a = k_weight[lane]; kw_b = k_weight[lane + 32]; }
    pdl_wait();
    const int heads = Hq + 2 * Hkv;
    const int head0 = (blockIdx.y * 4 + (threadIdx.x >> 5)) * kRopeHeadsPerWarp;
    if (head0 >= heads) return;
    uint32_t a[kRopeHeadsPerWarp], b[kRopeHeadsPerWarp];
#pragma unroll
    for (int h = 0; h < kRopeHeadsPerWarp; ++h) {
        const int head = head0 + h;
        if (head < heads) {
            const uint32_t* src = qkv + ((size_t)t * heads + head) * 64;
            a[h] = src[lane];
            b[h] = src[lane + 32];
        }
    }
    const float2 c = cos_t[(size_t)t * 32 + lane], sn = sin_t[(size_t)t * 32 + lane];
    int slot = Hkv ? slots[t] : -1;
    if (slot >= 0 && !slot_ok(slot, page_size, bounds)) slot = -1;
#pragma unroll
    for (int h = 0; h < kRopeHeadsPerWarp; ++h) {
        const int head = head0 + h;
        if (head >= heads) break;
        const bool is_q = head < Hq, is_k = !is_q && head < Hq + Hkv;
        uint32_t* dst;
        if (is_q) {
            dst = q_out + ((size_t)t * Hq + head) * 64;
        } else {
            if (slot < 0) continue;
            const int kvh = is_k ? head - Hq : head - Hq - Hkv;
            dst = (is_k ? k_pool : v_pool) + (((size_t)(slot / page_size) * Hkv + kvh) * page_size + slot % page_size) * 64;
        }
        if (!is_q && !is_k) {
            dst[lane] = a[h];
            dst[lane + 32] = b[h];
            continue;
        }
        float a0 = __uint_as_float(a[h] << 16), a1 = __uint_as_float(a[h] & 0xffff0000u);
        float b0 = __uint_as_float(b[h] << 16), b1 = __uint_as_float(b[h] & 0xffff0000u);
        const float2* w = is_q ? q_weight : k_weight;
        if (w) {
            const float inv = rsqrtf(warp_sum(a0 * a0 + a1 * a1 + b0 * b0 + b1 * b1) / 128.0f + eps);
            const float2 wa = is_q ? qw_a : kw_a, wb = is_q ? qw_b : kw_b;
            a0 *= inv * wa.x; a1 *= inv * wa.y; b0 *= inv * wb.x; b1 *= inv * wb.y;
        }
        const __nv_bfloat162 lo = __floats2bfloat162_rn(a0 * c.x - b0 * sn.x, a1 * c.y - b1 * sn.y);
        const __nv_bfloat162 hi = __floats2bfloat162_rn(b0 * c.x + a0 * sn.x, b1 * c.y + a1 * sn.y);
        dst[lane] = *reinterpret_cast<const uint32_t*>(&lo);
        dst[lane + 32] = *reinterpret_cast<const uint32_t*>(&hi);
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

// The same on 16-byte vectors of bfloat16 (inter % 8 == 0, 16-byte aligned rows).
__global__ void silu_mul_bf16x8_kernel(const uint4* __restrict__ gu, uint4* __restrict__ out, int inter8, size_t total8) {
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total8;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / inter8;
        const int i = (int)(idx - t * inter8);
        const uint4 gv = gu[t * 2 * inter8 + i], uv = gu[t * 2 * inter8 + inter8 + i];
        const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
        uint32_t r[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float g0 = __uint_as_float(gw[k] << 16), g1 = __uint_as_float(gw[k] & 0xffff0000u);
            const float u0 = __uint_as_float(uw[k] << 16), u1 = __uint_as_float(uw[k] & 0xffff0000u);
            const __nv_bfloat162 v = __floats2bfloat162_rn(g0 / (1.0f + expf(-g0)) * u0, g1 / (1.0f + expf(-g1)) * u1);
            r[k] = *reinterpret_cast<const uint32_t*>(&v);
        }
        out[idx] = make_uint4(r[0], r[1], r[2], r[3]);
    }
}

int block_for(int width) {
    int b = 32;
    while (b < 1024 && b * 4 < width) b <<= 1;
    return b;
}

// ids[dst[i]] = src_ids[src[i]]: token ids that an earlier step sampled go straight into this step's
// ids without passing through the host.
__global__ void move_ids_kernel(int* __restrict__ ids, const int* __restrict__ dst, const int* __restrict__ src,
                                const int* __restrict__ src_ids, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) ids[dst[i]] = src_ids[src[i]];
}

}  // namespace

// ids[dst[i]] = src_ids[src[i]] for i < n.  (The reference reads every sampled token back to the host and sends
// it down again with the next step: pulsar-core/src/runtime/engine.cpp:703-729, 573-600.)
PB_EXPORT int pb_move_ids(int* ids, const int* dst, const int* src, const int* src_ids, int n, cudaStream_t stream) {
    if (n <= 0) return 0;
    move_ids_kernel<<<(n + 127) / 128, 128, 0, stream>>>(ids, dst, src, src_ids, n);
    return launch_status();
}

namespace pb {
static PoolBounds g_pool_bounds = {0, nullptr};
PoolBounds pool_bounds_now() { return g_pool_bounds; }
}  // namespace pb

// 1 in a build with the bounds checks (see common.cuh), else 0.
PB_EXPORT int pb_bounds_checked(void) {
#ifdef PB_CHECK_BOUNDS
    return 1;
#else
    return 0;
#endif
}

// What the kernels launched from now on check page ids and slots against: a pool of n_pages pages, violations
// recorded in *error (a device word).  n_pages <= 0 or error null: unchecked.  Does nothing without the build flag.
PB_EXPORT void pb_set_pool_bounds(int n_pages, unsigned int* error) {
#ifdef PB_CHECK_BOUNDS
    pb::g_pool_bounds.n_pages = n_pages;
    pb::g_pool_bounds.error = error;
#else
    (void)n_pages;
    (void)error;
#endif
}

namespace {
struct WordList { const unsigned int* p[8]; };
__global__ void gather_words_kernel(WordList words, int n, int* out) {
    if ((int)threadIdx.x < n) out[threadIdx.x] = (int)*(volatile const unsigned int*)words.p[threadIdx.x];
}
}  // namespace

// out[i] = *words[i] for up to 8 device words, in the stream: the error words of the kernels with bounded waits,
// gathered so that one copy takes them to the host beside a step's results.
PB_EXPORT int pb_gather_words(const void* const* words, int n, int* out, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (n > 8) return PB_ERR_TOO_LARGE;
    WordList w;
    for (int i = 0; i < 8; ++i) w.p[i] = i < n ? (const unsigned int*)words[i] : nullptr;
    gather_words_kernel<<<1, 32, 0, stream>>>(w, n, out);
    return launch_status();
}

// x[i] = cap > 0 ? cap * tanh(x[i] * scale / cap) : x[i] * scale, in place, for n float32 values.
PB_EXPORT int pb_scale_cap(float* x, long long n, float scale, float cap, cudaStream_t stream) {
    if (n <= 0) return 0;
    long long blocks = (n + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    scale_cap_kernel<<<(int)blocks, 256, 0, stream>>>(x, (size_t)n, scale, cap);
    return launch_status();
}

// out[t] = table[ids[t]] * scale (float32 out; scale 1 for most architectures).
namespace {
// Block i serves sequence i of the step: it writes the page ids that the step brings for that sequence's row of the
// resident table, then copies the row's first `width` entries into the step's table.
__global__ void table_update_kernel(int* __restrict__ resident, int row_stride, const int* __restrict__ updates,
                                    const int* __restrict__ rows, int width, int* __restrict__ out) {
    const int i = blockIdx.x;
    const int row = rows[i];
    int* mine = resident + (size_t)row * row_stride;
    const int n = updates[0];
    for (int u = threadIdx.x; u < n; u += blockDim.x) {
        const int* t = updates + 1 + 3 * u;
        if (t[0] == row && t[1] >= 0 && t[1] < row_stride) mine[t[1]] = t[2];
    }
    __syncthreads();
    for (int j = threadIdx.x; j < width; j += blockDim.x) out[(size_t)i * width + j] = mine[j];
}
}  // namespace

// The device's resident block tables (one row of `row_stride` page ids per state slot): `updates` = the count, then
// (row, logical page, page id) triples that the step's requests gained; `rows` [n_seqs] = each sequence's row.
// out [n_seqs, width] receives the rows' first `width` entries: the block table the step's kernels read.
// width <= row_stride.  Entries beyond a request's pages hold whatever an earlier holder of the row left there.
PB_EXPORT int pb_table_update(int* resident, int row_stride, const int* updates, const int* rows, int n_seqs, int width, int* out,
                              cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (width <= 0 || width > row_stride) return PB_ERR_BAD_SIZE;
    table_update_kernel<<<n_seqs, 128, 0, stream>>>(resident, row_stride, updates, rows, width, out);
    return launch_status();
}

PB_EXPORT int pb_embed(int dtype, const void* table, const int* ids, float* out, int n, int width, int vocab, float scale,
                       cudaStream_t stream) {
    if (n <= 0) return 0;
    const int b = block_for(width);
    if (dtype == PB_F32) embed_kernel<float><<<n, b, 0, stream>>>((const float*)table, ids, out, width, vocab, scale);
    else if (dtype == PB_BF16) embed_kernel<__nv_bfloat16><<<n, b, 0, stream>>>((const __nv_bfloat16*)table, ids, out, width, vocab, scale);
    else return PB_ERR_BAD_DTYPE;
    return launch_status();
}

PB_EXPORT int pb_add_rmsnorm(int dtype, float* residual, const void* delta, const float* weight, void* out,
                             const int* rows, int n_out, int width, float eps, int write_back, cudaStream_t stream) {
    if (n_out <= 0) return 0;
    if (rows && write_back) return PB_ERR_BAD_SIZE;   // gathered rows are read-only
    if (dtype != PB_F32 && dtype != PB_BF16) return PB_ERR_BAD_DTYPE;
    const bool aligned = (((uintptr_t)residual | (uintptr_t)delta | (uintptr_t)weight | (uintptr_t)out) & 15) == 0;
    if (width % 4 == 0 && width <= 8192 && aligned) {
        const int vecs = width / 4;
        const int vpt = vecs <= 1024 ? 1 : 2;
        int threads = ((vecs + vpt - 1) / vpt + 31) / 32 * 32;
        if (dtype == PB_F32) {
            if (vpt == 1) return launch_pdl(add_rmsnorm_vec_kernel<float, 1>, n_out, threads, 0, stream, residual, (const float*)delta, weight, (float*)out, rows, width, eps, write_back);
            return launch_pdl(add_rmsnorm_vec_kernel<float, 2>, n_out, threads, 0, stream, residual, (const float*)delta, weight, (float*)out, rows, width, eps, write_back);
        }
        if (vpt == 1) return launch_pdl(add_rmsnorm_vec_kernel<__nv_bfloat16, 1>, n_out, threads, 0, stream, residual, (const __nv_bfloat16*)delta, weight, (__nv_bfloat16*)out, rows, width, eps, write_back);
        return launch_pdl(add_rmsnorm_vec_kernel<__nv_bfloat16, 2>, n_out, threads, 0, stream, residual, (const __nv_bfloat16*)delta, weight, (__nv_bfloat16*)out, rows, width, eps, write_back);
    }
    const int b = block_for(width);
    if (dtype == PB_F32)
        add_rmsnorm_kernel<float><<<n_out, b, 0, stream>>>(residual, (const float*)delta, weight, (float*)out, rows, width, eps, write_back);
    else
        add_rmsnorm_kernel<__nv_bfloat16><<<n_out, b, 0, stream>>>(residual, (const __nv_bfloat16*)delta, weight, (__nv_bfloat16*)out, rows, width, eps, write_back);
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
    if (dtype == PB_BF16 && D == 128 && rotary == 128) {
        dim3 fast_grid(n, (heads + warps * kRopeHeadsPerWarp - 1) / (warps * kRopeHeadsPerWarp));
        return launch_pdl(qk_norm_rope_write_bf16_d128_kernel, fast_grid, warps * 32, 0, stream, (const uint32_t*)qkv, (uint32_t*)q_out,
            (uint32_t*)k_pool, (uint32_t*)v_pool, slots, (const float2*)cos_t, (const float2*)sin_t, (const float2*)q_weight,
            (const float2*)k_weight, eps, Hq, Hkv, page_size, pb::pool_bounds_now());
    }
    dim3 grid(n, (heads + warps - 1) / warps);
    if (dtype == PB_F32)
        qk_norm_rope_write_kernel<float><<<grid, warps * 32, 0, stream>>>((const float*)qkv, (float*)q_out, (float*)k_pool, (float*)v_pool,
            slots, cos_t, sin_t, q_weight, k_weight, eps, Hq, Hkv, D, rotary, page_size, pb::pool_bounds_now());
    else if (dtype == PB_BF16)
        qk_norm_rope_write_kernel<__nv_bfloat16><<<grid, warps * 32, 0, stream>>>((const __nv_bfloat16*)qkv, (__nv_bfloat16*)q_out,
            (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, slots, cos_t, sin_t, q_weight, k_weight, eps, Hq, Hkv, D, rotary, page_size,
            pb::pool_bounds_now());
    else return PB_ERR_BAD_DTYPE;
    return launch_status();
}

PB_EXPORT int pb_silu_mul(int dtype, const void* gate_up, void* out, int n, int inter, cudaStream_t stream) {
    if (n <= 0) return 0;
    const size_t total = (size_t)n * inter;
    const int b = 256;
    size_t blocks = (total + b - 1) / b;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (dtype == PB_BF16 && inter % 8 == 0 && ((uintptr_t)gate_up & 15) == 0 && ((uintptr_t)out & 15) == 0) {
        size_t total8 = total / 8, blocks8 = (total8 + b - 1) / b;
        if (blocks8 > 148 * 16) blocks8 = 148 * 16;
        silu_mul_bf16x8_kernel<<<(int)blocks8, b, 0, stream>>>((const uint4*)gate_up, (uint4*)out, inter / 8, total8);
    } else if (dtype == PB_F32) silu_mul_kernel<float><<<(int)blocks, b, 0, stream>>>((const float*)gate_up, (float*)out, inter, total);
    else if (dtype == PB_BF16) silu_mul_kernel<__nv_bfloat16><<<(int)blocks, b, 0, stream>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter, total);
    else return PB_ERR_BAD_DTYPE;
    return launch_status();
}
