// Token selection on the device.
//
// Greedy rows (temperature <= 0) take the argmax of the raw logits, lowest index on
// ties.  Other rows draw from softmax(logits / temperature) restricted by top-k and
// top-p with the reference's meaning (pulsar-core/src/runtime/sampler.cpp:12-46):
// in descending order of probability a token survives iff fewer than k tokens are
// more probable and the mass of the more probable tokens is <= top_p (the token that
// crosses top_p stays).  The reference sorts the row.  Here the smallest surviving
// probability is found without a sort: "survives" is monotone in the probability, so the
// bit pattern of the threshold is fixed ten bits at a time from histograms (count and mass
// per bin of the probabilities' bit patterns; masses as 64-bit fixed point, so that the sums
// do not depend on the order of the atomic additions).  Tokens of equal probability survive or
// fall together.  The draw inverts the cumulative mass of the survivors, taken in index order,
// at u * (surviving mass); u in [0,1) comes from the request's own generator on the host, so a
// seed reproduces its tokens whatever else is batched.
//
// Every row is worked on by up to 32 blocks (a vocabulary of 150 thousand is 600 KB per row): one
// kernel for the slices' maxima and sums, three for the histograms (each block first reads the
// levels above it and decides their bins again, the same way), one for the survivors' masses per
// slice, whose last block per row draws the token.
#include "common.cuh"

#include <climits>

namespace {

using namespace pb;

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

// ---------------------------------------------------------------------------------------------
// Stochastic rows
constexpr int kSampleThreads = 256;
constexpr int kMaxSlices = 32;
constexpr int kBins = 1024;                       // ten bits of the probability's bit pattern per level
constexpr int kLevels = 3;                        // probabilities are <= 1.0 = 0x3F800000 < 2^30
constexpr float kMassScale = 281474976710656.0f;  // 2^48: masses as 64-bit fixed point

struct SampleWork {                               // device scratch of one call
    float2* part;                                 // [rows][slices]: maximum and sum of exp((x - maximum) / T) of a slice
    unsigned int* cnt;                            // [levels][rows][bins]
    unsigned long long* mass;                     // [levels][rows][bins]
    float* slice_mass;                            // [rows][slices]: mass of a slice above the threshold
    int* slice_ties;                              // [rows][slices]: tokens of a slice at the threshold
    unsigned int* tickets;                        // [rows]
};

struct RowParams {
    float inv_t, m, inv_z;
    int k;
    unsigned long long tp_q;
    bool use_k, use_p;
};

// Maximum and normaliser of a row from its slices' partial results, in slice order (every block gets the same bits).
__device__ __forceinline__ void row_softmax(const float2* part, int slices, float inv_t, float& m, float& inv_z) {
    m = -INFINITY;
    for (int s = 0; s < slices; ++s) m = fmaxf(m, part[s].x);
    float z = 0.0f;
    for (int s = 0; s < slices; ++s) z += part[s].y * expf((part[s].x - m) * inv_t);
    inv_z = 1.0f / z;
}

__device__ __forceinline__ RowParams row_params(int r, const float2* part, int slices, int vocab, const float* temperature,
                                                const int* top_k, const float* top_p) {
    RowParams p;
    p.inv_t = 1.0f / temperature[r];
    row_softmax(part + (size_t)r * slices, slices, p.inv_t, p.m, p.inv_z);
    p.k = top_k ? top_k[r] : 0;
    const float tp = top_p ? top_p[r] : 1.0f;
    p.use_k = p.k > 0 && p.k < vocab;
    p.use_p = tp > 0.0f && tp < 1.0f;
    p.tp_q = (unsigned long long)((double)tp * (double)kMassScale);
    return p;
}

__device__ __forceinline__ float prob(float x, const RowParams& p) { return expf((x - p.m) * p.inv_t) * p.inv_z; }

// The bin of one level that holds the threshold, given count and mass of everything above the level's range:
// the lowest bin b such that what lies above b (carried + the bins above it) passes "fewer than k and mass <= top_p".
// Adds what lies above that bin to the carried totals.  All threads of the block call it and get the same answer.
__device__ int pick_bin(const unsigned int* cnt, const unsigned long long* mass, const RowParams& p, unsigned int& carried_cnt,
                        unsigned long long& carried_mass, unsigned int* s_cnt, unsigned long long* s_mass, int* s_pick) {
    constexpr int kPer = kBins / kSampleThreads;
    const int t = threadIdx.x;
    unsigned int c = 0;
    unsigned long long m = 0;
#pragma unroll
    for (int i = 0; i < kPer; ++i) { c += cnt[t * kPer + i]; m += mass[t * kPer + i]; }
    __syncthreads();
    s_cnt[t] = c;
    s_mass[t] = m;
    if (t == 0) *s_pick = kBins;
    __syncthreads();
    // inclusive suffix sums over the threads' groups of bins
    for (int o = 1; o < kSampleThreads; o <<= 1) {
        const unsigned int c2 = t + o < kSampleThreads ? s_cnt[t + o] : 0;
        const unsigned long long m2 = t + o < kSampleThreads ? s_mass[t + o] : 0;
        __syncthreads();
        s_cnt[t] += c2;
        s_mass[t] += m2;
        __syncthreads();
    }
    // above the thread's highest bin: the groups after it
    unsigned int above_c = carried_cnt + (t + 1 < kSampleThreads ? s_cnt[t + 1] : 0);
    unsigned long long above_m = carried_mass + (t + 1 < kSampleThreads ? s_mass[t + 1] : 0);
    int mine = kBins;
#pragma unroll
    for (int i = kPer - 1; i >= 0; --i) {          // from the thread's highest bin down: `above` grows
        const int b = t * kPer + i;
        const bool ok = (!p.use_k || above_c < (unsigned int)p.k) && (!p.use_p || above_m <= p.tp_q);
        if (ok) mine = b;
        above_c += cnt[b];
        above_m += mass[b];
    }
    if (mine < kBins) atomicMin(s_pick, mine);
    __syncthreads();
    const int b = *s_pick;                          // exists: nothing above the top bin always passes
    // what lies above bin b: groups after b's group, and the bins above b inside its group
    const int gt = b / kPer;
    unsigned int add_c = gt + 1 < kSampleThreads ? s_cnt[gt + 1] : 0;
    unsigned long long add_m = gt + 1 < kSampleThreads ? s_mass[gt + 1] : 0;
    for (int i = b + 1; i < (gt + 1) * kPer; ++i) { add_c += cnt[i]; add_m += mass[i]; }
    carried_cnt += add_c;
    carried_mass += add_m;
    __syncthreads();
    return b;
}

__device__ __forceinline__ void slice_range(int vocab, int slices, int slice, int& begin, int& end) {
    const int per = (vocab + slices - 1) / slices;
    begin = slice * per;
    end = min(vocab, begin + per);
}

__global__ void __launch_bounds__(kSampleThreads)
sample_stats_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temperature, SampleWork w) {
    __shared__ float scratch[32];
    const int r = blockIdx.y, slices = gridDim.x;
    const float temp = temperature[r];
    if (!(temp > 0.0f)) return;
    const float inv_t = 1.0f / temp;
    const float* row = logits + (size_t)r * vocab;
    int begin, end;
    slice_range(vocab, slices, blockIdx.x, begin, end);
    float m = -INFINITY;
    for (int i = begin + threadIdx.x; i < end; i += kSampleThreads) m = fmaxf(m, row[i]);
    m = warp_max(m);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) scratch[warp] = m;
    __syncthreads();
    m = scratch[0];
    for (int i = 1; i < kSampleThreads / 32; ++i) m = fmaxf(m, scratch[i]);
    float z = 0.0f;
    if (m > -INFINITY)
        for (int i = begin + threadIdx.x; i < end; i += kSampleThreads) z += expf((row[i] - m) * inv_t);
    z = block_sum(z, scratch);
    if (threadIdx.x == 0) w.part[(size_t)r * slices + blockIdx.x] = make_float2(m, z);
}

// Level L (0 = the highest ten bits): histogram of the probabilities whose higher bits equal the bins picked above.
template <int LEVEL>
__global__ void __launch_bounds__(kSampleThreads)
sample_hist_kernel(const float* __restrict__ logits, int rows, int vocab, const float* __restrict__ temperature,
                   const int* __restrict__ top_k, const float* __restrict__ top_p, SampleWork w) {
    __shared__ unsigned int h_cnt[kBins];
    __shared__ unsigned long long h_mass[kBins];
    __shared__ unsigned int s_cnt[kSampleThreads];
    __shared__ unsigned long long s_mass[kSampleThreads];
    __shared__ int s_pick;
    const int r = blockIdx.y, slices = gridDim.x;
    if (!(temperature[r] > 0.0f)) return;
    const RowParams p = row_params(r, w.part, slices, vocab, temperature, top_k, top_p);
    if (!p.use_k && !p.use_p) return;
    unsigned int carried_cnt = 0;
    unsigned long long carried_mass = 0;
    unsigned int prefix = 0;                      // the bins picked on the levels above, as the high bits
#pragma unroll
    for (int l = 0; l < LEVEL; ++l) {
        const size_t at = ((size_t)l * rows + r) * kBins;
        const int b = pick_bin(w.cnt + at, w.mass + at, p, carried_cnt, carried_mass, s_cnt, s_mass, &s_pick);
        prefix = (prefix << 10) | (unsigned int)b;
    }
    for (int i = threadIdx.x; i < kBins; i += kSampleThreads) { h_cnt[i] = 0; h_mass[i] = 0; }
    __syncthreads();
    const float* row = logits + (size_t)r * vocab;
    int begin, end;
    slice_range(vocab, slices, blockIdx.x, begin, end);
    constexpr int kShift = 10 * (kLevels - 1 - LEVEL);
    for (int i = begin + threadIdx.x; i < end; i += kSampleThreads) {
        const float q = prob(row[i], p);
        const unsigned int key = __float_as_uint(q);
        if (LEVEL == 0 || (key >> (kShift + 10)) == prefix) {
            const unsigned int bin = (key >> kShift) & (kBins - 1);
            atomicAdd(&h_cnt[bin], 1u);
            atomicAdd(&h_mass[bin], (unsigned long long)(q * kMassScale));
        }
    }
    __syncthreads();
    const size_t at = ((size_t)LEVEL * rows + r) * kBins;
    for (int i = threadIdx.x; i < kBins; i += kSampleThreads)
        if (h_cnt[i]) {
            atomicAdd(w.cnt + at + i, h_cnt[i]);
            atomicAdd(w.mass + at + i, h_mass[i]);
        }
}

// Mass of the survivors of every slice, in index order; the last block of a row to finish inverts the
// cumulative mass at u * (surviving mass).
__global__ void __launch_bounds__(kSampleThreads)
sample_draw_kernel(const float* __restrict__ logits, int rows, int vocab, const float* __restrict__ temperature,
                   const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ uniform,
                   SampleWork w, int* __restrict__ out) {
    __shared__ unsigned int s_cnt[kSampleThreads];
    __shared__ unsigned long long s_mass[kSampleThreads];
    __shared__ float scan_s[kSampleThreads];
    __shared__ int s_pick, s_ties;
    __shared__ bool s_last;
    __shared__ Best best_s[32];
    const int r = blockIdx.y, slices = gridDim.x;
    if (!(temperature[r] > 0.0f)) return;
    const RowParams p = row_params(r, w.part, slices, vocab, temperature, top_k, top_p);
    // threshold: the smallest surviving probability.  allow: how many of the tokens whose probability EQUALS it
    // survive, the first ones in index order: a sort keeps exactly k tokens and the nucleus rule looks at the mass
    // strictly before each token (pulsar-core/src/runtime/sampler.cpp:30-40), so equal probabilities at the cut are
    // not all in or all out.
    float threshold = 0.0f;
    int allow = INT_MAX;
    if (p.use_k || p.use_p) {
        unsigned int carried_cnt = 0, bits = 0;
        unsigned long long carried_mass = 0;
        for (int l = 0; l < kLevels; ++l) {
            const size_t at = ((size_t)l * rows + r) * kBins;
            bits = (bits << 10) | (unsigned int)pick_bin(w.cnt + at, w.mass + at, p, carried_cnt, carried_mass, s_cnt, s_mass, &s_pick);
        }
        threshold = __uint_as_float(bits);
        // carried_*: count and mass of what lies strictly above the threshold (fewer than k, mass <= top_p)
        if (p.use_k) allow = p.k - (int)carried_cnt;
        if (p.use_p) {
            const unsigned long long each = (unsigned long long)(threshold * kMassScale);
            const unsigned long long room = p.tp_q >= carried_mass ? p.tp_q - carried_mass : 0;
            const unsigned long long by_mass = each > 0 ? room / each + 1 : (unsigned long long)INT_MAX;
            if (by_mass < (unsigned long long)allow) allow = (int)by_mass;
        }
        if (allow < 1) allow = 1;
    }
    const float* row = logits + (size_t)r * vocab;
    // thread t owns a contiguous range of the slice's indices.  ``ties_before``: tokens at the threshold in the
    // slices before this one.  With target < 0 only the slice's mass above the threshold (s_mass[0]) and its
    // number of tokens at the threshold (s_ties) are wanted.
    auto scan_slice = [&](int slice, float target, float before_slice, int ties_before) -> int {
        int begin, end;
        slice_range(vocab, slices, slice, begin, end);
        const int per = (end - begin + kSampleThreads - 1) / kSampleThreads;
        const int b0 = min(end, begin + (int)threadIdx.x * per), e0 = min(end, b0 + per);
        float mine = 0.0f;
        int my_ties = 0;
        for (int i = b0; i < e0; ++i) {
            const float q = prob(row[i], p);
            if (q > threshold) mine += q;
            else if (q == threshold) ++my_ties;
        }
        __syncthreads();
        scan_s[threadIdx.x] = mine;
        s_cnt[threadIdx.x] = (unsigned int)my_ties;
        __syncthreads();
        if (threadIdx.x == 0) {      // serial prefix over the partials: fixed order, negligible time
            float run = before_slice;
            int ties = ties_before;
            const bool count_ties = target >= 0.0f;
            for (int t = 0; t < kSampleThreads; ++t) {
                const int n = (int)s_cnt[t];
                const int in = count_ties ? max(0, min(n, allow - min(ties, allow))) : 0;
                const float v = scan_s[t] + (float)in * threshold;
                scan_s[t] = run;
                s_cnt[t] = (unsigned int)ties;             // ties before thread t's range
                run += v;
                ties += n;
            }
            s_mass[0] = (unsigned long long)__float_as_uint(run);
            s_ties = ties - ties_before;
            s_pick = -1;
        }
        __syncthreads();
        if (target < 0.0f) return -1;
        const float before = scan_s[threadIdx.x];
        int ties = (int)s_cnt[threadIdx.x];
        const float my_mass = mine + (float)max(0, min(my_ties, allow - min(ties, allow))) * threshold;
        if (my_mass > 0.0f && target >= before && target < before + my_mass) {
            float run = before;
            int chosen = -1, last = -1;
            for (int i = b0; i < e0; ++i) {
                const float q = prob(row[i], p);
                const bool in = q > threshold || (q == threshold && ties++ < allow);
                if (in) {
                    last = i;
                    run += q;
                    if (target < run) { chosen = i; break; }
                }
            }
            s_pick = chosen >= 0 ? chosen : last;
        }
        __syncthreads();
        return s_pick;
    };
    scan_slice(blockIdx.x, -1.0f, 0.0f, 0);
    if (threadIdx.x == 0) {
        w.slice_mass[(size_t)r * slices + blockIdx.x] = __uint_as_float((unsigned int)s_mass[0]);
        w.slice_ties[(size_t)r * slices + blockIdx.x] = s_ties;
        __threadfence();
        s_last = atomicAdd(w.tickets + r, 1u) == (unsigned int)slices - 1;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // the row's last block: which slice holds the target, then which token
    auto slice_total = [&](int s, int ties_before) -> float {
        const float above = *reinterpret_cast<volatile float*>(w.slice_mass + (size_t)r * slices + s);
        const int n = *reinterpret_cast<volatile int*>(w.slice_ties + (size_t)r * slices + s);
        return above + (float)max(0, min(n, allow - min(ties_before, allow))) * threshold;
    };
    float total = 0.0f;
    int ties = 0;
    for (int s = 0; s < slices; ++s) {
        total += slice_total(s, ties);
        ties += *reinterpret_cast<volatile int*>(w.slice_ties + (size_t)r * slices + s);
    }
    const float target = uniform[r] * total;
    float before = 0.0f;
    int slice = -1;
    ties = 0;
    for (int s = 0; s < slices; ++s) {
        const float v = slice_total(s, ties);
        if (v > 0.0f && target < before + v) { slice = s; break; }
        before += v;
        ties += *reinterpret_cast<volatile int*>(w.slice_ties + (size_t)r * slices + s);
    }
    int pick = slice >= 0 ? scan_slice(slice, target, before, ties) : -1;
    if (pick < 0) pick = block_argmax(row, vocab, best_s);      // rounding left the target past the last survivor
    if (threadIdx.x == 0) {
        out[r] = pick;
        w.tickets[r] = 0;
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

// KiB of device scratch that pb_sample needs for `rows` rows.
PB_EXPORT int pb_sample_workspace(int rows) {
    if (rows <= 0) return 0;
    const long long r = rows;
    const long long bytes = r * kMaxSlices * sizeof(float2) + (long long)kLevels * r * kBins * (sizeof(unsigned int) + sizeof(unsigned long long)) +
                            r * kMaxSlices * (sizeof(float) + sizeof(int)) + r * sizeof(unsigned int) + 256;
    return (int)((bytes + 1023) / 1024);
}

// Rows with temperature <= 0 take the argmax; the others draw from softmax(logits / temperature) restricted by
// top_k (null or <= 0: off) and top_p (null or outside (0, 1): off) at uniform[r] in [0, 1).  `workspace`:
// pb_sample_workspace(rows) KiB, 16-byte aligned; `keys`: rows 64-bit words.  any_greedy = 0 says that no row is
// greedy (the argmax kernels are left out).
PB_EXPORT int pb_sample(const float* logits, int rows, int vocab, const float* temperature, const int* top_k,
                        const float* top_p, const float* uniform, int any_greedy, void* workspace,
                        unsigned long long* keys, int* out, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0 || rows > 65535) return PB_ERR_BAD_SIZE;
    if (!temperature || !uniform || !workspace || (((uintptr_t)workspace) & 15)) return PB_ERR_BAD_SIZE;
    if (any_greedy) {
        const int rc = pb_argmax(logits, rows, vocab, keys, out, stream);       // stochastic rows are overwritten below
        if (rc != 0) return rc;
    }
    int slices = (vocab + 2047) / 2048;
    if (slices > kMaxSlices) slices = kMaxSlices;
    SampleWork w;
    unsigned char* at = static_cast<unsigned char*>(workspace);
    w.mass = reinterpret_cast<unsigned long long*>(at);
    at += (size_t)kLevels * rows * kBins * sizeof(unsigned long long);
    w.cnt = reinterpret_cast<unsigned int*>(at);
    at += (size_t)kLevels * rows * kBins * sizeof(unsigned int);
    w.tickets = reinterpret_cast<unsigned int*>(at);
    at += ((size_t)rows * sizeof(unsigned int) + 15) / 16 * 16;
    const size_t zeroed = (size_t)(at - static_cast<unsigned char*>(workspace));
    w.part = reinterpret_cast<float2*>(at);
    at += (size_t)rows * kMaxSlices * sizeof(float2);
    w.slice_mass = reinterpret_cast<float*>(at);
    at += (size_t)rows * kMaxSlices * sizeof(float);
    w.slice_ties = reinterpret_cast<int*>(at);
    cudaError_t rc = cudaMemsetAsync(workspace, 0, zeroed, stream);
    if (rc != cudaSuccess) return (int)rc;
    const dim3 grid(slices, rows);
    sample_stats_kernel<<<grid, kSampleThreads, 0, stream>>>(logits, vocab, temperature, w);
    if (top_k || top_p) {
        sample_hist_kernel<0><<<grid, kSampleThreads, 0, stream>>>(logits, rows, vocab, temperature, top_k, top_p, w);
        sample_hist_kernel<1><<<grid, kSampleThreads, 0, stream>>>(logits, rows, vocab, temperature, top_k, top_p, w);
        sample_hist_kernel<2><<<grid, kSampleThreads, 0, stream>>>(logits, rows, vocab, temperature, top_k, top_p, w);
    }
    sample_draw_kernel<<<grid, kSampleThreads, 0, stream>>>(logits, rows, vocab, temperature, top_k, top_p, uniform, w, out);
    return launch_status();
}
