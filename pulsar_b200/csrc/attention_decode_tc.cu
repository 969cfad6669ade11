// Paged decode attention on the tensor cores for bfloat16 pages with head size 64 or 128
// and up to 16 query heads per kv head.
//
// One block per (split of the keys, kv head, sequence).  The group's query heads fill the
// rows of one 16-row MMA tile (as the reference packs them,
// pulsar-core/src/kernels/paged_attention.cu:101-203); keys and values stream through a
// three-stage cp.async pipeline of 64-key tiles, gathered page by page through the block
// table into XOR-swizzled shared memory, so that ldmatrix reads are free of bank
// conflicts.  Each of the four warps owns 16 keys of a tile: S = Q K^T with
// mma.m16n8k16, an online softmax in float32 on the accumulator fragments (exp2f on
// scores pre-multiplied by scale*log2(e)), P rounded to bfloat16 as the A operand of
// O += P V.  The warps' partial results are merged through shared memory and written in
// the layout of the split kernel (attention_decode.cu), whose combine kernel finishes.
//
// This kernel exists for memory bandwidth: a decode step reads every cached key and value
// once, and what limits it is the number of bytes in flight per SM, not arithmetic.
#include "mma_common.cuh"

#include <cstdlib>

namespace {

using namespace pb;

constexpr int kTile = 64;        // keys per pipeline stage
constexpr int kStages = 3;
constexpr int kWarps = 4;

template <int D>
__global__ void __launch_bounds__(kWarps * 32, 2)
decode_tc_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pool, const bf16* __restrict__ v_pool,
                 float* __restrict__ partial, const int* __restrict__ block_table, int table_stride,
                 const int* __restrict__ kv_len, int Hq, int Hkv, int page_shift, float scale, int window, int n_splits,
                 bf16* __restrict__ out, unsigned int* __restrict__ tickets, int evict_first, const PoolBounds bounds) {
    constexpr int kTileBytes = kTile * D * 2;
    constexpr int kKSteps = D / 16;                   // k-steps of Q K^T
    constexpr int kNTiles = D / 8;                    // n-tiles of P V
    extern __shared__ __align__(128) unsigned char smem[];
    // [stage][K tile | V tile]; after the main loop the same memory holds the warps' partial results
    const uint32_t smem_base = smem_u32(smem);

    const int split = blockIdx.x, kvh = blockIdx.y, s = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int G = Hq / Hkv;
    const int p = kv_len[s] - 1;
    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const int n_keys = p - lo + 1;
    int chunk = (n_keys + n_splits - 1) / n_splits;
    chunk = (chunk + kTile - 1) / kTile * kTile;
    const int begin = lo + split * chunk;
    const int end = min(p + 1, begin + chunk);        // keys [begin, end)
    const int* table = block_table + (size_t)s * table_stride;
    const int tile0 = begin / kTile;                  // tiles are aligned to absolute key indices (whole pages)
    const int n_tiles = begin < end ? (end - 1) / kTile - tile0 + 1 : 0;

    // Every cached key and value is read by exactly one block of a step: with the policy the lines leave L2 first.
    const uint64_t policy = evict_first ? l2_policy_evict_first() : 0;
    auto issue_tile = [&](int tile_index, int stage) {
        const uint32_t k_dst = smem_base + stage * 2 * kTileBytes;
        load_kv_tile<D, kWarps * 32>(k_dst, k_dst + kTileBytes, k_pool, v_pool, table, (tile0 + tile_index) * kTile, begin,
                                     end - 1, kvh, Hkv, page_shift, tid, policy, bounds);
    };

    // The kernel before this one writes only the newest key and value (position p).  Tiles that lie wholly
    // below p are requested before waiting for it; kv_len and the block table come from the host.
    bool early[kStages - 1];
#pragma unroll
    for (int i = 0; i < kStages - 1; ++i) {
        early[i] = i < n_tiles && (tile0 + i) * kTile + kTile - 1 < p;
        if (early[i]) { issue_tile(i, i); cp_async_commit(); }
    }
    pdl_wait();

    // Q fragments: rows = query heads of the group (zero beyond G), straight from global memory.
    uint32_t qa[kKSteps][4];
    {
        const bf16* q0 = q + ((size_t)s * Hq + (size_t)kvh * G) * D;
#pragma unroll
        for (int ks = 0; ks < kKSteps; ++ks) {
            const int c0 = ks * 16 + 2 * t;
            qa[ks][0] = g < G ? *reinterpret_cast<const uint32_t*>(q0 + (size_t)g * D + c0) : 0u;
            qa[ks][1] = g + 8 < G ? *reinterpret_cast<const uint32_t*>(q0 + (size_t)(g + 8) * D + c0) : 0u;
            qa[ks][2] = g < G ? *reinterpret_cast<const uint32_t*>(q0 + (size_t)g * D + c0 + 8) : 0u;
            qa[ks][3] = g + 8 < G ? *reinterpret_cast<const uint32_t*>(q0 + (size_t)(g + 8) * D + c0 + 8) : 0u;
        }
    }

    float o[kNTiles][4];
#pragma unroll
    for (int i = 0; i < kNTiles; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};     // rows g and g + 8
    const float sl2 = scale * kLog2e;

#pragma unroll
    for (int i = 0; i < kStages - 1; ++i) {
        if (early[i]) continue;                       // requested above (early tiles come first, so the order of groups holds)
        if (i < n_tiles) issue_tile(i, i);
        cp_async_commit();
    }
    for (int it = 0; it < n_tiles; ++it) {
        cp_async_wait<kStages - 2>();
        __syncthreads();                              // tile `it` has landed; stage (it-1) % kStages is free
        if (it + kStages - 1 < n_tiles) issue_tile(it + kStages - 1, (it + kStages - 1) % kStages);
        cp_async_commit();

        const int stage = it % kStages;
        const uint32_t k_s = smem_base + stage * 2 * kTileBytes, v_s = k_s + kTileBytes;
        const int key_base = (tile0 + it) * kTile + warp * 16;            // this warp's 16 keys
        if (key_base >= end || key_base + 16 <= begin) continue;           // nothing of this warp's is in range

        // S = Q K^T for 16 heads x 16 keys (two n-tiles of 8 keys)
        float sc[2][4];
#pragma unroll
        for (int n = 0; n < 2; ++n) { sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.0f; }
#pragma unroll
        for (int ks = 0; ks < kKSteps; ++ks) {
            // matrices: (keys 0-7, d 0-7), (keys 0-7, d 8-15), (keys 8-15, d 0-7), (keys 8-15, d 8-15)
            uint32_t kb[4];
            const int row = warp * 16 + (lane & 7) + ((lane >> 4) << 3);
            const int c = ks * 2 + ((lane >> 3) & 1);
            ldmatrix_x4(kb, k_s + tile_offset<D>(row, c));
            mma_bf16(sc[0], qa[ks], kb[0], kb[1]);
            mma_bf16(sc[1], qa[ks], kb[2], kb[3]);
        }
        // mask and scale; thread holds keys key_base + n*8 + 2t + {0,1} for rows g (c0,c1) and g+8 (c2,c3)
        float tmax[2] = {-INFINITY, -INFINITY};
        if (key_base >= begin && key_base + 16 <= end) {                   // every key of the warp is in range
#pragma unroll
            for (int n = 0; n < 2; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    sc[n][e] *= sl2;
                    tmax[e >> 1] = fmaxf(tmax[e >> 1], sc[n][e]);
                }
        } else {
#pragma unroll
            for (int n = 0; n < 2; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = key_base + n * 8 + 2 * t + (e & 1);
                    const float v = (key >= begin && key < end) ? sc[n][e] * sl2 : -INFINITY;
                    sc[n][e] = v;
                    tmax[e >> 1] = fmaxf(tmax[e >> 1], v);
                }
        }
        float corr[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float mx = tmax[r];
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m_run[r], mx);                      // finite: at least one key of the warp is in range
            corr[r] = exp2f(m_run[r] - m_new);
            m_run[r] = m_new;
            l_run[r] *= corr[r];
        }
        uint32_t pa[4];
        {
            float pv[2][4];
#pragma unroll
            for (int n = 0; n < 2; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    pv[n][e] = exp2f(sc[n][e] - m_run[e >> 1]);
                    l_run[e >> 1] += pv[n][e];
                }
            pa[0] = pack_bf16(pv[0][0], pv[0][1]);
            pa[1] = pack_bf16(pv[0][2], pv[0][3]);
            pa[2] = pack_bf16(pv[1][0], pv[1][1]);
            pa[3] = pack_bf16(pv[1][2], pv[1][3]);
        }
#pragma unroll
        for (int i = 0; i < kNTiles; ++i) {
            o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1];
        }
        // O += P V: V^T fragments by transposing ldmatrix over [16 keys][16 d] blocks
#pragma unroll
        for (int i = 0; i < kNTiles; i += 2) {
            // matrices: (keys 0-7, d i*8..), (keys 8-15, d i*8..), (keys 0-7, d (i+1)*8..), (keys 8-15, d (i+1)*8..)
            uint32_t vb[4];
            const int row = warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
            const int c = i + (lane >> 4);
            ldmatrix_x4_trans(vb, v_s + tile_offset<D>(row, c));
            mma_bf16(o[i], pa, vb[0], vb[1]);
            mma_bf16(o[i + 1], pa, vb[2], vb[3]);
        }
    }
    cp_async_wait<0>();
    __syncthreads();
    pdl_trigger();

    // Merge the four warps (each saw a quarter of the keys) and write the split's partial.
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    float* o_s = reinterpret_cast<float*>(smem);            // [kWarps][16][D]
    float* m_s = o_s + kWarps * 16 * D;                      // [kWarps][16]
    float* l_s = m_s + kWarps * 16;
#pragma unroll
    for (int i = 0; i < kNTiles; ++i) {
        const int d = i * 8 + 2 * t;
        o_s[(warp * 16 + g) * D + d] = o[i][0];
        o_s[(warp * 16 + g) * D + d + 1] = o[i][1];
        o_s[(warp * 16 + g + 8) * D + d] = o[i][2];
        o_s[(warp * 16 + g + 8) * D + d + 1] = o[i][3];
    }
    if (t == 0) {
        m_s[warp * 16 + g] = m_run[0]; m_s[warp * 16 + g + 8] = m_run[1];
        l_s[warp * 16 + g] = l_run[0]; l_s[warp * 16 + g + 8] = l_run[1];
    }
    __syncthreads();
    const int stride = D + 2;
    // With `tickets` the kernel finishes the job itself: a single split writes the result at once; of
    // several splits the one that draws the last ticket of its (sequence, kv head) merges all partials
    // in split order (no block waits for another).  Without tickets a combine kernel follows.
    const bool direct = tickets != nullptr && n_splits == 1;
    for (int i = tid; i < G * D; i += kWarps * 32) {
        const int h = i / D, d = i - h * D;
        float m_all = -INFINITY;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) m_all = fmaxf(m_all, m_s[w * 16 + h]);
        float acc = 0.0f, l_all = 0.0f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            const float f = (m_s[w * 16 + h] == -INFINITY) ? 0.0f : exp2f(m_s[w * 16 + h] - m_all);
            acc += o_s[(w * 16 + h) * D + d] * f;
            l_all += l_s[w * 16 + h] * f;
        }
        if (direct) {
            out[((size_t)s * Hq + (size_t)kvh * G + h) * D + d] = __float2bfloat16_rn(l_all > 0.0f ? acc / l_all : 0.0f);
        } else {
            float* dst = partial + (((size_t)s * Hq + (size_t)kvh * G + h) * n_splits + split) * stride;
            __stcg(dst + d, acc);
            if (d == 0) { __stcg(dst + D, m_all * kLn2); __stcg(dst + D + 1, l_all); }   // maximum back in natural-log units
        }
    }
    if (tickets == nullptr || direct) return;
    __shared__ unsigned int ticket_s;
    __threadfence();
    __syncthreads();
    if (tid == 0) ticket_s = atomicAdd(tickets + (size_t)s * Hkv + kvh, 1u);
    __syncthreads();
    if (ticket_s != (unsigned)(n_splits - 1)) return;
    __threadfence();
    float* w_s = reinterpret_cast<float*>(smem);            // [G][n_splits] weights, then [G] sums (the tiles are done with)
    float* lsum_s = w_s + G * n_splits;
    const float* base = partial + ((size_t)s * Hq + (size_t)kvh * G) * n_splits * stride;
    if (tid < G) {
        const float* hb = base + (size_t)tid * n_splits * stride;
        float m_all = -INFINITY;
        for (int i = 0; i < n_splits; ++i) m_all = fmaxf(m_all, __ldcg(hb + i * stride + D));
        float l_all = 0.0f;
        for (int i = 0; i < n_splits; ++i) {
            const float m = __ldcg(hb + i * stride + D);
            const float wgt = (m > -INFINITY) ? expf(m - m_all) : 0.0f;
            w_s[tid * n_splits + i] = wgt;
            l_all += __ldcg(hb + i * stride + D + 1) * wgt;
        }
        lsum_s[tid] = l_all;
    }
    if (tid == 0) tickets[(size_t)s * Hkv + kvh] = 0;        // ready for the next launch
    __syncthreads();
    for (int i = tid; i < G * D; i += kWarps * 32) {
        const int h = i / D, d = i - h * D;
        const float* hb = base + (size_t)h * n_splits * stride;
        float acc = 0.0f;
        for (int sp = 0; sp < n_splits; ++sp) acc = fmaf(__ldcg(hb + sp * stride + d), w_s[h * n_splits + sp], acc);
        out[((size_t)s * Hq + (size_t)kvh * G + h) * D + d] = __float2bfloat16_rn(lsum_s[h] > 0.0f ? acc / lsum_s[h] : 0.0f);
    }
}

template <int D>
int launch_tc(const void* q, const void* k_pool, const void* v_pool, float* partial, const int* block_table,
              int table_stride, const int* kv_len, int n_seqs, int Hq, int Hkv, int page_size, float scale, int window,
              int n_splits, void* out, unsigned int* tickets, cudaStream_t stream) {
    const int page_shift = log2_exact(page_size);
    constexpr int pipeline = kStages * 2 * kTile * D * 2;
    constexpr int merge = (kWarps * 16 * D + 2 * kWarps * 16) * 4;
    constexpr int smem = pipeline > merge ? pipeline : merge;
    static bool configured = false;
    if (!configured) {
        cudaError_t rc = cudaFuncSetAttribute(decode_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (rc != cudaSuccess) return (int)rc;
        configured = true;
    }
    static const int evict_first = [] { const char* v = getenv("PULSAR_DECODE_EVICT_FIRST"); return (v && v[0] == '0' && v[1] == 0) ? 0 : 1; }();
    dim3 grid(n_splits, Hkv, n_seqs);
    return launch_pdl(decode_tc_kernel<D>, grid, kWarps * 32, smem, stream, (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool,
                      partial, block_table, table_stride, kv_len, Hq, Hkv, page_shift, scale, window, n_splits, (bf16*)out, tickets, evict_first,
                      pool_bounds_now());
}

}  // namespace

PB_EXPORT int pb_decode_combine(int dtype, const float* partial, void* out, int rows, int D, int n_splits, cudaStream_t stream);

// 1 if pb_paged_attention_decode_tc takes these sizes (else the split kernel of attention_decode.cu serves).
PB_EXPORT int pb_decode_tc_supported(int dtype, int Hq, int Hkv, int D, int page_size) {
    if (dtype != PB_BF16 || Hkv <= 0 || Hq % Hkv || Hq / Hkv > 16) return 0;
    if (D != 64 && D != 128) return 0;
    if (log2_exact(page_size) < 0 || page_size > kTile) return 0;      // a power of two up to the tile
    return 1;
}

// Same arguments and scratch as pb_paged_attention_decode.
PB_EXPORT int pb_paged_attention_decode_tc(int dtype, const void* q, const void* k_pool, const void* v_pool, void* out,
                                           float* partial, const int* block_table, int table_stride, const int* kv_len,
                                           int n_seqs, int Hq, int Hkv, int D, int page_size, float scale, int window,
                                           int n_splits, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (!pb_decode_tc_supported(dtype, Hq, Hkv, D, page_size) || n_splits <= 0) return PB_ERR_BAD_SIZE;
    if (Hkv > 65535 || n_seqs > 65535) return PB_ERR_TOO_LARGE;
    int rc;
    if (D == 64)
        rc = launch_tc<64>(q, k_pool, v_pool, partial, block_table, table_stride, kv_len, n_seqs, Hq, Hkv, page_size, scale,
                           window, n_splits, nullptr, nullptr, stream);
    else
        rc = launch_tc<128>(q, k_pool, v_pool, partial, block_table, table_stride, kv_len, n_seqs, Hq, Hkv, page_size, scale,
                            window, n_splits, nullptr, nullptr, stream);
    if (rc != 0) return rc;
    return pb_decode_combine(dtype, partial, out, n_seqs * Hq, D, n_splits, stream);
}

// The same in one launch: the split that finishes last merges.  `tickets`: n_seqs * Hkv 32-bit words that are
// zero before the first launch (every launch leaves them zero); n_splits <= 64.
PB_EXPORT int pb_paged_attention_decode_tc_fused(int dtype, const void* q, const void* k_pool, const void* v_pool, void* out,
                                                 float* partial, unsigned int* tickets, const int* block_table,
                                                 int table_stride, const int* kv_len, int n_seqs, int Hq, int Hkv, int D,
                                                 int page_size, float scale, int window, int n_splits, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (!pb_decode_tc_supported(dtype, Hq, Hkv, D, page_size) || n_splits <= 0 || tickets == nullptr) return PB_ERR_BAD_SIZE;
    if (Hkv > 65535 || n_seqs > 65535 || n_splits > 64) return PB_ERR_TOO_LARGE;
    if (D == 64)
        return launch_tc<64>(q, k_pool, v_pool, partial, block_table, table_stride, kv_len, n_seqs, Hq, Hkv, page_size, scale,
                             window, n_splits, out, tickets, stream);
    return launch_tc<128>(q, k_pool, v_pool, partial, block_table, table_stride, kv_len, n_seqs, Hq, Hkv, page_size, scale,
                          window, n_splits, out, tickets, stream);
}
