// Token selection on the device: one block per logits row.
//
// Greedy rows (temperature <= 0) take the argmax of the raw logits, lowest index on
// ties.  Other rows draw from softmax(logits / temperature) restricted by top-k and
// top-p with the reference's meaning (pulsar-core/src/runtime/sampler.cpp:12-46):
// in descending order of probability a token survives iff fewer than k tokens are
// more probable and the mass of the more probable tokens is <= top_p (the token that
// crosses top_p stays).  The reference sorts the row; here the smallest surviving
// probability is found by bisection over float bit patterns, which needs no sort:
// "survives" is monotone in the probability.  Tokens of equal probability survive or
// fall together.  The draw inverts the cumulative mass of the survivors, taken in
// index order, at u * (surviving mass); u in [0,1) comes from the request's own
// generator on the host, so a seed reproduces its tokens whatever else is batched.
#include "common.cuh"

namespace {

using namespace pb;

constexpr int kThreads = 1024;

struct Best { float v; int i; };

__device__ __forceinline__ Best better(Best a, Best b) {
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

__device__ int block_argmax(const float* row, int vocab, Best* sh) {
    Best best = {-INFINITY, 0x7fffffff};
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) best = better(best, Best{row[i], i});
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best other = {__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
        best = better(best, other);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) sh[warp] = best;
    __syncthreads();
    if (warp == 0) {
        best = (lane < (int)(blockDim.x >> 5)) ? sh[lane] : Best{-INFINITY, 0x7fffffff};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            Best other = {__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
            best = better(best, other);
        }
        if (lane == 0) sh[0] = best;
    }
    __syncthreads();
    const int idx = sh[0].i;
    return idx == 0x7fffffff ? 0 : idx;
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = (lane < (int)(blockDim.x >> 5)) ? scratch[lane] : -INFINITY;
    return warp_max(t);
}

__global__ void __launch_bounds__(kThreads)
sample_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ uniform,
              int* __restrict__ out) {
    __shared__ Best best_s[32];
    __shared__ float scratch[32];
    __shared__ float scan_s[kThreads];
    __shared__ int pick_s;
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * vocab;
    const float temp = temperature ? temperature[r] : 0.0f;
    if (!(temp > 0.0f)) {
        const int idx = block_argmax(row, vocab, best_s);
        if (threadIdx.x == 0) out[r] = idx;
        return;
    }
    const float inv_t = 1.0f / temp;
    float m = -INFINITY;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) m = fmaxf(m, row[i]);
    m = block_max(m, scratch);
    float z = 0.0f;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) z += expf((row[i] - m) * inv_t);
    z = block_sum(z, scratch);
    const float inv_z = 1.0f / z;

    const int k = top_k ? top_k[r] : 0;
    const float tp = top_p ? top_p[r] : 1.0f;
    const bool use_k = k > 0 && k < vocab, use_p = tp > 0.0f && tp < 1.0f;
    float threshold = 0.0f;
    if (use_k || use_p) {
        // Smallest float tau such that count(p > tau) < k and mass(p > tau) <= top_p.
        unsigned lo = 0u, hi = __float_as_uint(1.0f);     // ok(hi): nothing exceeds probability 1
        while (lo < hi) {
            const unsigned mid = lo + ((hi - lo) >> 1);
            const float tau = __uint_as_float(mid);
            float cnt = 0.0f, mass = 0.0f;
            for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
                const float p = expf((row[i] - m) * inv_t) * inv_z;
                if (p > tau) { cnt += 1.0f; mass += p; }
            }
            cnt = block_sum(cnt, scratch);
            mass = block_sum(mass, scratch);
            const bool ok = (!use_k || cnt < (float)k) && (!use_p || mass <= tp);
            if (ok) hi = mid; else lo = mid + 1;
        }
        threshold = __uint_as_float(lo);
    }
    // Survivors in index order: thread t owns a contiguous range of indices.
    const int per = (vocab + blockDim.x - 1) / blockDim.x;
    const int begin = threadIdx.x * per, end = min(vocab, begin + per);
    float mine = 0.0f;
    for (int i = begin; i < end; ++i) {
        const float p = expf((row[i] - m) * inv_t) * inv_z;
        if (p >= threshold) mine += p;
    }
    scan_s[threadIdx.x] = mine;
    if (threadIdx.x == 0) pick_s = -1;
    __syncthreads();
    if (threadIdx.x == 0) {      // serial prefix over 1024 partials: fixed order, negligible time
        float run = 0.0f;
        for (int t = 0; t < (int)blockDim.x; ++t) { const float v = scan_s[t]; scan_s[t] = run; run += v; }
        scratch[0] = run;
    }
    __syncthreads();
    const float target = uniform[r] * scratch[0];
    const float before = scan_s[threadIdx.x];
    if (mine > 0.0f && target >= before && target < before + mine) {
        float run = before;
        int chosen = -1, last = -1;
        for (int i = begin; i < end; ++i) {
            const float p = expf((row[i] - m) * inv_t) * inv_z;
            if (p >= threshold) {
                last = i;
                run += p;
                if (target < run) { chosen = i; break; }
            }
        }
        pick_s = chosen >= 0 ? chosen : last;
    }
    __syncthreads();
    if (pick_s < 0) {            // rounding left the target past the last survivor: take the most probable
        const int idx = block_argmax(row, vocab, best_s);
        if (threadIdx.x == 0) out[r] = idx;
    } else if (threadIdx.x == 0) {
        out[r] = pick_s;
    }
}

// Greedy rows over many blocks: every block reduces a slice of the row to (value, index) and
// merges it into the row's 64-bit key with atomicMax.  The key orders by value, then by
// lower index: high word = float bits made monotone, low word = ~index.
__device__ __forceinline__ unsigned long long argmax_key(float v, int i) {
    uint32_t b = __float_as_uint(v);
    b = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
    return ((unsigned long long)b << 32) | (uint32_t)(~(uint32_t)i);
}

__global__ void __launch_bounds__(256)
argmax_partial_kernel(const float* __restrict__ logits, int vocab, unsigned long long* __restrict__ keys) {
    __shared__ Best best_s[32];
    const int r = blockIdx.y;
    const float* row = logits + (size_t)r * vocab;
    const int per = (vocab + gridDim.x - 1) / gridDim.x;
    const int begin = blockIdx.x * per, end = min(vocab, begin + per);
    Best best = {-INFINITY, 0x7fffffff};
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) best = better(best, Best{row[i], i});
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best other = {__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
        best = better(best, other);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) best_s[warp] = best;
    __syncthreads();
    if (warp == 0) {
        best = (lane < (int)(blockDim.x >> 5)) ? best_s[lane] : Best{-INFINITY, 0x7fffffff};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            Best other = {__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
            best = better(best, other);
        }
        if (lane == 0 && best.i != 0x7fffffff) atomicMax(keys + r, argmax_key(best.v, best.i));
    }
}

__global__ void argmax_finish_kernel(const unsigned long long* __restrict__ keys, int* __restrict__ out, int rows) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r < rows) out[r] = keys[r] ? (int)(~(uint32_t)(keys[r] & 0xffffffffu)) : 0;
}

}  // namespace

// Greedy selection for every row with many blocks per row.  `keys` is scratch of `rows`
// 64-bit words (cleared here, on the stream).
PB_EXPORT int pb_argmax(const float* logits, int rows, int vocab, unsigned long long* keys, int* out, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0 || rows > 65535) return PB_ERR_BAD_SIZE;
    cudaError_t rc = cudaMemsetAsync(keys, 0, sizeof(unsigned long long) * rows, stream);
    if (rc != cudaSuccess) return (int)rc;
    int slices = (vocab + 4095) / 4096;
    if (slices > 64) slices = 64;
    argmax_partial_kernel<<<dim3(slices, rows), 256, 0, stream>>>(logits, vocab, keys);
    argmax_finish_kernel<<<(rows + 127) / 128, 128, 0, stream>>>(keys, out, rows);
    return launch_status();
}

// temperature, top_k, top_p may be null (greedy / off); uniform may be null only when every row is greedy.
PB_EXPORT int pb_sample(const float* logits, int rows, int vocab, const float* temperature, const int* top_k,
                        const float* top_p, const float* uniform, int* out, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) return PB_ERR_BAD_SIZE;
    if (temperature && !uniform) return PB_ERR_BAD_SIZE;
    sample_kernel<<<rows, kThreads, 0, stream>>>(logits, vocab, temperature, top_k, top_p, uniform, out);
    return launch_status();
}
