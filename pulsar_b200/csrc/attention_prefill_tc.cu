// Paged attention for prompt portions on the tensor cores: causal, ragged batch (portions
// of any length beside single tokens), optional window, grouped heads, bfloat16 pages with
// head size 64 or 128.
//
// One block of four warps per (tile of 64 query tokens of one sequence, query head).  The
// query tile is loaded once and kept as MMA A fragments; keys and values stream through a
// two-stage cp.async pipeline of 64-key tiles gathered page by page through the block
// table into XOR-swizzled shared memory.  Each warp owns 16 query rows: S = Q K^T by
// mma.m16n8k16, online softmax in float32 on the accumulator fragments (exp2f of scores
// pre-multiplied by scale*log2(e)), P rounded to bfloat16 as the A operand of O += P V.
// Key tiles above the diagonal or below the window are never loaded; a warp skips tiles
// none of its rows can see.  The heaviest tiles (ends of long portions) are launched first.
//
// Query token t of sequence s (rows cu_q[s]..cu_q[s+1]) sits at position
// kv_len[s] - q_len + (t - cu_q[s]): a portion of a prompt attends everything its request
// already has in the cache plus its own causal part, which is what chunked prefill and
// mixed batches need (pulsar-core/inc/pulsar/ops.hpp:106-111).
//
// Role in the reference: pulsar-core/inc/pulsar/kernels/paged_prefill.cuh:35-346
// (attn_prefill_tc_kernel, 16-query tiles, tile list built on the host) and the rotate
// pre-pass pulsar-core/src/kernels/paged_prefill.cu:28-60, which this engine does not need
// because keys are stored rotated.
#include "mma_common.cuh"

namespace {

using namespace pb;

constexpr int kBM = 64;          // query rows per block
constexpr int kBN = 64;          // keys per pipeline stage
constexpr int kWarps = 4;

// 2^x by the special-function unit (ex2.approx: relative error 2^-22, 2^-inf = 0).
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int D>
__global__ void __launch_bounds__(kWarps * 32, 2)
prefill_tc_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pool, const bf16* __restrict__ v_pool,
                  bf16* __restrict__ out, const int* __restrict__ block_table, int table_stride,
                  const int* __restrict__ cu_q, const int* __restrict__ kv_len, int n_seqs, int Hq, int Hkv,
                  int page_shift, float scale, int window, const PoolBounds bounds) {
    constexpr int kChunks = D / 8;
    constexpr int kTileBytes = kBN * D * 2;
    constexpr int kKSteps = D / 16;
    constexpr int kNTiles = D / 8;
    extern __shared__ __align__(128) unsigned char smem[];
    const uint32_t smem_base = smem_u32(smem);            // [2 stages][K tile | V tile]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int head = blockIdx.y;
    const int kvh = head / (Hq / Hkv);

    // Which sequence and which of its query tiles (heaviest first: reverse order).
    int tile = gridDim.x - 1 - blockIdx.x;
    int s = 0, q0 = 0, q_len = 0;
    for (; s < n_seqs; ++s) {
        q0 = cu_q[s];
        q_len = cu_q[s + 1] - q0;
        const int nt = (q_len + kBM - 1) / kBM;
        if (tile < nt) break;
        tile -= nt;
    }
    if (s >= n_seqs) return;
    const int m0 = tile * kBM;
    const int rows = min(kBM, q_len - m0);                 // valid query rows of this tile
    const int ctx0 = kv_len[s] - q_len;                    // position of the sequence's first new token
    const int pos_first = ctx0 + m0, pos_last = ctx0 + m0 + rows - 1;
    const int lo = (window > 0 && pos_first - window + 1 > 0) ? pos_first - window + 1 : 0;
    const int kt0 = lo / kBN, n_tiles = pos_last / kBN - kt0 + 1;
    const int* table = block_table + (size_t)s * table_stride;

    auto issue_kv = [&](int tile_index, int stage) {
        const uint32_t k_dst = smem_base + stage * 2 * kTileBytes;
        load_kv_tile<D, kWarps * 32>(k_dst, k_dst + kTileBytes, k_pool, v_pool, table, (kt0 + tile_index) * kBN, lo, pos_last,
                                     kvh, Hkv, page_shift, tid, 0, bounds);
    };

    // Q tile through the second stage's K buffer into registers, while the first K/V tile loads.
    {
        const uint32_t q_dst = smem_base + 2 * kTileBytes;
#pragma unroll
        for (int i = 0; i < kBM * kChunks / (kWarps * 32); ++i) {
            const int idx = i * kWarps * 32 + tid;
            const int row = idx / kChunks, c = idx % kChunks;
            const bool ok = row < rows;
            const bf16* src = q + ((size_t)(q0 + m0 + (ok ? row : 0)) * Hq + head) * D + c * 8;
            cp_async16(q_dst + tile_offset<D>(row, c), src, ok);
        }
        cp_async_commit();
        issue_kv(0, 0);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
    }
    uint32_t qa[kKSteps][4];
    {
        const uint32_t q_s = smem_base + 2 * kTileBytes;
        const int row = warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
#pragma unroll
        for (int ks = 0; ks < kKSteps; ++ks) ldmatrix_x4(qa[ks], q_s + tile_offset<D>(row, ks * 2 + (lane >> 4)));
    }
    __syncthreads();                                       // the Q buffer becomes stage 1

    float o[kNTiles][4];
#pragma unroll
    for (int i = 0; i < kNTiles; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    const float sl2 = scale * kLog2e;
    // positions of this thread's two rows (rows beyond the tile's end take the last valid one: results unused)
    const int r0 = min(warp * 16 + g, rows - 1), r1 = min(warp * 16 + g + 8, rows - 1);
    const int pos0 = pos_first + r0, pos1 = pos_first + r1;
    const int wpos_first = pos_first + min(warp * 16, rows - 1), wpos_last = pos_first + min(warp * 16 + 15, rows - 1);

    for (int it = 0; it < n_tiles; ++it) {
        if (it + 1 < n_tiles) issue_kv(it + 1, (it + 1) & 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();                                   // tile `it` has landed

        const int stage = it & 1;
        const uint32_t k_s = smem_base + stage * 2 * kTileBytes, v_s = k_s + kTileBytes;
        const int key0 = (kt0 + it) * kBN;
        const bool active = warp * 16 < rows && key0 <= wpos_last &&
                            (window <= 0 || key0 + kBN - 1 > wpos_first - window);
        if (active) {
            float sc[kBN / 8][4];
#pragma unroll
            for (int n = 0; n < kBN / 8; ++n) { sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.0f; }
#pragma unroll
            for (int ks = 0; ks < kKSteps; ++ks) {
#pragma unroll
                for (int nn = 0; nn < kBN / 16; ++nn) {
                    uint32_t kb[4];
                    const int row = nn * 16 + (lane & 7) + ((lane >> 4) << 3);
                    ldmatrix_x4(kb, k_s + tile_offset<D>(row, ks * 2 + ((lane >> 3) & 1)));
                    mma_bf16(sc[2 * nn], qa[ks], kb[0], kb[1]);
                    mma_bf16(sc[2 * nn + 1], qa[ks], kb[2], kb[3]);
                }
            }
            float tmax[2] = {-INFINITY, -INFINITY};
            // every row of the warp sees every key of the tile: below the diagonal and inside the window
            const bool all_visible = key0 + kBN - 1 <= wpos_first && (window <= 0 || key0 > wpos_last - window);
            if (all_visible) {
#pragma unroll
                for (int n = 0; n < kBN / 8; ++n)
#pragma unroll
                    for (int e = 0; e < 4; ++e) tmax[e >> 1] = fmaxf(tmax[e >> 1], sc[n][e]);
            } else {
#pragma unroll
                for (int n = 0; n < kBN / 8; ++n)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int key = key0 + n * 8 + 2 * t + (e & 1);
                        const int pos = (e >> 1) ? pos1 : pos0;
                        const bool vis = key <= pos && (window <= 0 || key > pos - window);
                        const float v = vis ? sc[n][e] : -INFINITY;
                        sc[n][e] = v;
                        tmax[e >> 1] = fmaxf(tmax[e >> 1], v);
                    }
            }
            // Running maxima are kept on the raw scores (sl2 > 0 keeps the order); the scale enters
            // only the exponent: p = 2^(s * sl2 - m * sl2), one multiply-add and one ex2 per score.
            float corr[2], neg_ms[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                float mx = tmax[r];
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                const float m_new = fmaxf(m_run[r], mx);
                const float m_safe = (m_new == -INFINITY) ? 0.0f : m_new;     // a row that has seen no key yet
                corr[r] = ex2((m_run[r] - m_safe) * sl2);
                neg_ms[r] = -m_safe * sl2;
                m_run[r] = m_new;
                l_run[r] *= corr[r];
            }
            if (__any_sync(0xffffffffu, corr[0] != 1.0f || corr[1] != 1.0f)) {    // the maxima rarely move after the first tiles
#pragma unroll
                for (int i = 0; i < kNTiles; ++i) {
                    o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1];
                }
            }
#pragma unroll
            for (int kk = 0; kk < kBN / 16; ++kk) {
                uint32_t pa[4];
                float pv[2][4];
#pragma unroll
                for (int n = 0; n < 2; ++n)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        pv[n][e] = ex2(fmaf(sc[2 * kk + n][e], sl2, neg_ms[e >> 1]));
                        l_run[e >> 1] += pv[n][e];
                    }
                pa[0] = pack_bf16(pv[0][0], pv[0][1]);
                pa[1] = pack_bf16(pv[0][2], pv[0][3]);
                pa[2] = pack_bf16(pv[1][0], pv[1][1]);
                pa[3] = pack_bf16(pv[1][2], pv[1][3]);
#pragma unroll
                for (int i = 0; i < kNTiles; i += 2) {
                    uint32_t vb[4];
                    const int row = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
                    ldmatrix_x4_trans(vb, v_s + tile_offset<D>(row, i + (lane >> 4)));
                    mma_bf16(o[i], pa, vb[0], vb[1]);
                    mma_bf16(o[i + 1], pa, vb[2], vb[3]);
                }
            }
        }
        __syncthreads();                                   // everyone is done with this stage before it is refilled
    }
    cp_async_wait<0>();

    // Normalise, round, and store 16 bytes at a time through the warp's own shared-memory rows.
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    const float inv0 = l_run[0] > 0.0f ? 1.0f / l_run[0] : 0.0f, inv1 = l_run[1] > 0.0f ? 1.0f / l_run[1] : 0.0f;
    unsigned char* w_s = smem + warp * 16 * D * 2;          // [16 rows][D] bf16, swizzled like the tiles
#pragma unroll
    for (int i = 0; i < kNTiles; ++i) {
        const uint32_t lo_off = tile_offset<D>(g, i) + (2 * t) * 2, hi_off = tile_offset<D>(g + 8, i) + (2 * t) * 2;
        *reinterpret_cast<uint32_t*>(w_s + lo_off) = pack_bf16(o[i][0] * inv0, o[i][1] * inv0);
        *reinterpret_cast<uint32_t*>(w_s + hi_off) = pack_bf16(o[i][2] * inv1, o[i][3] * inv1);
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 16 * kChunks / 32; ++i) {
        const int idx = i * 32 + lane;
        const int row = idx / kChunks, c = idx % kChunks;
        const int m = warp * 16 + row;
        if (m < rows) {
            const uint4 v = *reinterpret_cast<const uint4*>(w_s + tile_offset<D>(row, c));
            *reinterpret_cast<uint4*>(out + ((size_t)(q0 + m0 + m) * Hq + head) * D + c * 8) = v;
        }
    }
}

template <int D>
int launch_prefill(const void* q, const void* k_pool, const void* v_pool, void* out, const int* block_table,
                   int table_stride, const int* cu_q, const int* kv_len, int n_seqs, int n_q_tiles, int Hq, int Hkv,
                   int page_size, float scale, int window, cudaStream_t stream) {
    constexpr int smem = 2 * 2 * kBN * D * 2;
    const int page_shift = log2_exact(page_size);
    static bool configured = false;
    if (!configured) {
        cudaError_t rc = cudaFuncSetAttribute(prefill_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (rc != cudaSuccess) return (int)rc;
        configured = true;
    }
    dim3 grid(n_q_tiles, Hq);
    prefill_tc_kernel<D><<<grid, kWarps * 32, smem, stream>>>((const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool,
                                                              (bf16*)out, block_table, table_stride, cu_q, kv_len, n_seqs,
                                                              Hq, Hkv, page_shift, scale, window, pool_bounds_now());
    return launch_status();
}

}  // namespace

// Query rows per block: the caller sizes the grid as the sum over sequences of ceil(q_len / this).
PB_EXPORT int pb_prefill_tc_tile(void) { return kBM; }

PB_EXPORT int pb_prefill_tc_supported(int dtype, int Hq, int Hkv, int D, int page_size) {
    if (dtype != PB_BF16 || Hkv <= 0 || Hq % Hkv) return 0;
    if (D != 64 && D != 128) return 0;
    if (log2_exact(page_size) < 0 || page_size > kBN) return 0;         // a power of two up to the tile
    return 1;
}

// q, out [N, Hq, D]; n_q_tiles = sum over sequences of ceil(q_len / pb_prefill_tc_tile()).
PB_EXPORT int pb_paged_attention_prefill_tc(int dtype, const void* q, const void* k_pool, const void* v_pool, void* out,
                                            const int* block_table, int table_stride, const int* cu_q, const int* kv_len,
                                            int n_seqs, int n_q_tiles, int Hq, int Hkv, int D, int page_size, float scale,
                                            int window, cudaStream_t stream) {
    if (n_seqs <= 0 || n_q_tiles <= 0) return 0;
    if (!pb_prefill_tc_supported(dtype, Hq, Hkv, D, page_size)) return PB_ERR_BAD_SIZE;
    if (Hq > 65535) return PB_ERR_TOO_LARGE;
    if (D == 64)
        return launch_prefill<64>(q, k_pool, v_pool, out, block_table, table_stride, cu_q, kv_len, n_seqs, n_q_tiles, Hq, Hkv,
                                  page_size, scale, window, stream);
    return launch_prefill<128>(q, k_pool, v_pool, out, block_table, table_stride, cu_q, kv_len, n_seqs, n_q_tiles, Hq, Hkv,
                               page_size, scale, window, stream);
}
