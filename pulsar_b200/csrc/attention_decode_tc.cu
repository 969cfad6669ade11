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
// The kernel can also take over what otherwise runs as a kernel of its own before it: with a QkvFuse it reads the
// step's raw q/k/v rows, applies the per-head RMSNorm and the rotation to its group's query heads as it loads them,
// and the block whose keys include the newest position does the same for that position's key, writes key and value
// into their page, and only then asks for the tile that holds them.  One launch less in a chain of dependent
// launches, each of which costs more than a microsecond whatever it does.
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

// The step's projected rows, still without norm and rotation: [n_seqs][(Hq + 2 Hkv) * D] bfloat16, query heads first,
// then key heads, then value heads.  The whole head rotates (pairs i, i + D / 2).  qkv null: q is ready and the newest
// key and value are in their page.
struct QkvFuse {
    const bf16* qkv;
    const float* q_weight;      // [D] or null (no norm)
    const float* k_weight;
    const float* cos_t;         // [n_seqs][D / 2]
    const float* sin_t;
    const int* slots;           // [n_seqs] slot of the newest position: page * page_size + offset; negative: not cached
    bf16* k_out;                // the pools, writable
    bf16* v_out;
    float eps;
    int page_size;
};

__device__ __forceinline__ void unpack_bf16(uint32_t v, float& lo, float& hi) {
    lo = __uint_as_float(v << 16);
    hi = __uint_as_float(v & 0xffff0000u);
}

template <int D>
__global__ void __launch_bounds__(kWarps * 32, 2)
decode_tc_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pool, const bf16* __restrict__ v_pool,
                 float* __restrict__ partial, const int* __restrict__ block_table, int table_stride,
                 const int* __restrict__ kv_len, int Hq, int Hkv, int page_shift, float scale, int window, int n_splits,
                 bf16* __restrict__ out, unsigned int* __restrict__ tickets, int evict_first /* bit 0: the L2 hint; bits 4-6: tiles asked of L2 ahead */,
                 const PoolBounds bounds,
                 const QkvFuse fuse) {
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
    const uint64_t policy = (evict_first & 1) ? l2_policy_evict_first() : 0;
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
    const int ahead = (evict_first >> 4) & 7;           // tiles beyond the two in flight that L2 is asked for
    for (int i = 0; i < ahead; ++i)
        if (kStages - 1 + i < n_tiles)
            prefetch_kv_tile_l2<D>(k_pool, v_pool, table, (tile0 + kStages - 1 + i) * kTile, begin, end - 1, kvh, Hkv, page_shift, tid, bounds);
    pdl_wait();

    // Q fragments: rows = query heads of the group (zero beyond G), straight from global memory.
    uint32_t qa[kKSteps][4];
    {
        const bf16* q0 = fuse.qkv != nullptr ? fuse.qkv + (size_t)s * (Hq + 2 * Hkv) * D + (size_t)kvh * G * D
                                             : q + ((size_t)s * Hq + (size_t)kvh * G) * D;
#pragma unroll
        for (int ks = 0; ks < kKSteps; ++ks) {
            const int c0 = ks * 16 + 2 * t;
            qa[ks][0] = g < G ? *reinterpret_cast<const uint32_t*>(q0 + (size_t)g * D + c0) : 0u;
            qa[ks][1] = g + 8 < G ? *reinterpret_cast<const uint32_t*>(q0 + (size_t)(g + 8) * D + c0) : 0u;
            qa[ks][2] = g < G ? *reinterpret_cast<const uint32_t*>(q0 + (size_t)g * D + c0 + 8) : 0u;
            qa[ks][3] = g + 8 < G ? *reinterpret_cast<const uint32_t*>(q0 + (size_t)(g + 8) * D + c0 + 8) : 0u;
        }
    }
    if (fuse.qkv != nullptr) {
        // Rows g (registers 0, 2) and g + 8 (registers 1, 3); the four threads of a row hold it whole.  RMSNorm in
        // float32, then the rotation of the pairs (c, c + D / 2), which lie kKSteps / 2 k-steps apart in one thread.
        float inv[2] = {1.0f, 1.0f};
        if (fuse.q_weight != nullptr) {
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                float ss = 0.0f;
#pragma unroll
                for (int ks = 0; ks < kKSteps; ++ks) {
                    float a0, a1, b0, b1;
                    unpack_bf16(qa[ks][r], a0, a1);
                    unpack_bf16(qa[ks][r + 2], b0, b1);
                    ss += a0 * a0 + a1 * a1 + b0 * b0 + b1 * b1;
                }
                ss += __shfl_xor_sync(0xffffffffu, ss, 1);
                ss += __shfl_xor_sync(0xffffffffu, ss, 2);
                inv[r] = rsqrtf(ss / (float)D + fuse.eps);
            }
        }
        const float* cos_row = fuse.cos_t + (size_t)s * (D / 2);
        const float* sin_row = fuse.sin_t + (size_t)s * (D / 2);
#pragma unroll
        for (int ks = 0; ks < kKSteps / 2; ++ks) {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int c = ks * 16 + 2 * t + 8 * half;
                const float2 cs = *reinterpret_cast<const float2*>(cos_row + c), sn = *reinterpret_cast<const float2*>(sin_row + c);
                float2 w_lo = make_float2(1.0f, 1.0f), w_hi = make_float2(1.0f, 1.0f);
                if (fuse.q_weight != nullptr) {
                    w_lo = *reinterpret_cast<const float2*>(fuse.q_weight + c);
                    w_hi = *reinterpret_cast<const float2*>(fuse.q_weight + c + D / 2);
                }
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    const int reg = half * 2 + r;
                    float a0, a1, b0, b1;
                    unpack_bf16(qa[ks][reg], a0, a1);
                    unpack_bf16(qa[ks + kKSteps / 2][reg], b0, b1);
                    if (fuse.q_weight != nullptr) {
                        a0 *= inv[r] * w_lo.x; a1 *= inv[r] * w_lo.y; b0 *= inv[r] * w_hi.x; b1 *= inv[r] * w_hi.y;
                    }
                    qa[ks][reg] = pack_bf16(a0 * cs.x - b0 * sn.x, a1 * cs.y - b1 * sn.y);
                    qa[ks + kKSteps / 2][reg] = pack_bf16(b0 * cs.x + a0 * sn.x, b1 * cs.y + a1 * sn.y);
                }
            }
        }
        // The newest key and value: the block whose keys include position p brings them into their page before it
        // asks for the tile that holds them (what a block wrote before a barrier, its later copies read).
        if (begin <= p && p < end) {
            int slot = fuse.slots[s];
            if (slot >= 0 && !slot_ok(slot, fuse.page_size, bounds)) slot = -1;
            if (slot >= 0) {
                constexpr int kHalf = D / 4;                      // 32-bit words in half a head
                const size_t row = (((size_t)(slot / fuse.page_size) * Hkv + kvh) * fuse.page_size + slot % fuse.page_size) * (D / 2);
                const uint32_t* src = reinterpret_cast<const uint32_t*>(fuse.qkv + (size_t)s * (Hq + 2 * Hkv) * D);
                if (warp == 0) {
                    const uint32_t* k_src = src + (size_t)(Hq + kvh) * (D / 2);
                    const bool has = lane < kHalf;
                    float a0, a1, b0, b1;
                    unpack_bf16(has ? k_src[lane] : 0u, a0, a1);
                    unpack_bf16(has ? k_src[lane + kHalf] : 0u, b0, b1);
                    if (fuse.k_weight != nullptr) {
                        const float k_inv = rsqrtf(warp_sum(a0 * a0 + a1 * a1 + b0 * b0 + b1 * b1) / (float)D + fuse.eps);
                        if (has) {
                            const float2 wa = reinterpret_cast<const float2*>(fuse.k_weight)[lane];
                            const float2 wb = reinterpret_cast<const float2*>(fuse.k_weight)[lane + kHalf];
                            a0 *= k_inv * wa.x; a1 *= k_inv * wa.y; b0 *= k_inv * wb.x; b1 *= k_inv * wb.y;
                        }
                    }
                    if (has) {
                        const float2 cs = reinterpret_cast<const float2*>(cos_row)[lane], sn = reinterpret_cast<const float2*>(sin_row)[lane];
                        uint32_t* dst = reinterpret_cast<uint32_t*>(fuse.k_out) + row;
                        dst[lane] = pack_bf16(a0 * cs.x - b0 * sn.x, a1 * cs.y - b1 * sn.y);
                        dst[lane + kHalf] = pack_bf16(b0 * cs.x + a0 * sn.x, b1 * cs.y + a1 * sn.y);
                    }
                } else if (warp == 1) {
                    const uint32_t* v_src = src + (size_t)(Hq + Hkv + kvh) * (D / 2);
                    uint32_t* dst = reinterpret_cast<uint32_t*>(fuse.v_out) + row;
                    for (int i = lane; i < D / 2; i += 32) dst[i] = v_src[i];
                }
            }
            __syncthreads();
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
        if (ahead > 0 && it + kStages - 1 + ahead < n_tiles)
            prefetch_kv_tile_l2<D>(k_pool, v_pool, table, (tile0 + it + kStages - 1 + ahead) * kTile, begin, end - 1, kvh, Hkv, page_shift, tid, bounds);

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
              int n_splits, void* out, unsigned int* tickets, cudaStream_t stream, const QkvFuse fuse = QkvFuse{}) {
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
    // With fewer blocks than SMs (a lone sequence) the two tiles a block has in flight are not enough to hide the
    // memory's latency: such a launch also asks L2 for the two tiles behind them (2.828 against 2.858 ms per step of one
    // sequence).  With more blocks that costs time (3.626 against 3.538 ms at 8 sequences, 10.31 against 9.49 at 64).
    // PULSAR_DECODE_AHEAD=n forces n tiles for every launch.
    static const int forced_ahead = [] { const char* a = getenv("PULSAR_DECODE_AHEAD"); return a ? (atoi(a) < 0 ? 0 : atoi(a) > 7 ? 7 : atoi(a)) : -1; }();
    static const int sms = [] {
        int dev = 0, v = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) v = 0;
        return v > 0 ? v : 148;
    }();
    static const int evict_flag = [] { const char* v = getenv("PULSAR_DECODE_EVICT_FIRST"); return (v && v[0] == '0' && v[1] == 0) ? 0 : 1; }();
    const int ahead = forced_ahead >= 0 ? forced_ahead : ((long long)n_splits * Hkv * n_seqs <= sms ? 2 : 0);
    const int evict_first = evict_flag | (ahead << 4);
    dim3 grid(n_splits, Hkv, n_seqs);
    return launch_pdl(decode_tc_kernel<D>, grid, kWarps * 32, smem, stream, (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool,
                      partial, block_table, table_stride, kv_len, Hq, Hkv, page_shift, scale, window, n_splits, (bf16*)out, tickets, evict_first,
                      pool_bounds_now(), fuse);
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

// The same attention for a step of single tokens whose rows come straight from the q/k/v product: qkv [n_seqs]
// [(Hq + 2 Hkv) * D] bfloat16 (query, key, value heads in this order).  The kernel applies the per-head RMSNorm
// (q_weight, k_weight float32 [D], or null for none; eps) and the rotation of the whole head (cos_t, sin_t float32
// [n_seqs][D / 2]) to the queries and to the newest key, and writes that key and the value to slots[s] of their
// pools before it reads them: what pb_qk_norm_rope_write does in a launch of its own.  tickets null: the splits are
// merged by pb_decode_combine; else as pb_paged_attention_decode_tc_fused.
PB_EXPORT int pb_paged_attention_decode_tc_qkv(int dtype, const void* qkv, const float* q_weight, const float* k_weight,
                                               const float* cos_t, const float* sin_t, float eps, const int* slots,
                                               void* k_pool, void* v_pool, void* out, float* partial, unsigned int* tickets,
                                               const int* block_table, int table_stride, const int* kv_len, int n_seqs, int Hq,
                                               int Hkv, int D, int page_size, float scale, int window, int n_splits,
                                               cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (!pb_decode_tc_supported(dtype, Hq, Hkv, D, page_size) || n_splits <= 0) return PB_ERR_BAD_SIZE;
    if (qkv == nullptr || cos_t == nullptr || sin_t == nullptr || slots == nullptr) return PB_ERR_BAD_SIZE;
    if ((((uintptr_t)cos_t | (uintptr_t)sin_t | (uintptr_t)q_weight | (uintptr_t)k_weight) & 7) != 0) return PB_ERR_BAD_SIZE;
    if (Hkv > 65535 || n_seqs > 65535 || (tickets != nullptr && n_splits > 64)) return PB_ERR_TOO_LARGE;
    QkvFuse fuse{};
    fuse.qkv = (const bf16*)qkv;
    fuse.q_weight = q_weight;
    fuse.k_weight = k_weight;
    fuse.cos_t = cos_t;
    fuse.sin_t = sin_t;
    fuse.slots = slots;
    fuse.k_out = (bf16*)k_pool;
    fuse.v_out = (bf16*)v_pool;
    fuse.eps = eps;
    fuse.page_size = page_size;
    int rc;
    if (D == 64)
        rc = launch_tc<64>(nullptr, k_pool, v_pool, partial, block_table, table_stride, kv_len, n_seqs, Hq, Hkv, page_size, scale,
                           window, n_splits, tickets ? out : nullptr, tickets, stream, fuse);
    else
        rc = launch_tc<128>(nullptr, k_pool, v_pool, partial, block_table, table_stride, kv_len, n_seqs, Hq, Hkv, page_size, scale,
                            window, n_splits, tickets ? out : nullptr, tickets, stream, fuse);
    if (rc != 0 || tickets != nullptr) return rc;
    return pb_decode_combine(dtype, partial, out, n_seqs * Hq, D, n_splits, stream);
}
