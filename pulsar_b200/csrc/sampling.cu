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

}  // namespace

// temperature, top_k, top_p may be null (greedy / off); uniform may be null only when every row is greedy.
PB_EXPORT int pb_sample(const float* logits, int rows, int vocab, const float* temperature, const int* top_k,
                        const float* top_p, const float* uniform, int* out, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) return PB_ERR_BAD_SIZE;
    if (temperature && !uniform) return PB_ERR_BAD_SIZE;
    sample_kernel<<<rows, kThreads, 0, stream>>>(logits, vocab, temperature, top_k, top_p, uniform, out);
    return launch_status();
}
