// Paged attention for prompt portions on the fifth-generation tensor cores: causal, ragged
// batch, optional window, grouped heads, bfloat16 pages, head size 128.
//
// A persistent grid of one block per SM (192 KB of shared memory, all 512 tensor-memory columns: two
// S tiles and two O tiles) walks over work items, each a tile of 128 query tokens of one sequence
// and one query head.  Roles inside a block:
//   warps 0-3   softmax: thread r owns query row r (tensor-memory lane r).  It reads its row of
//               S = Q K^T from tensor memory (tcgen05.ld), keeps the running maximum and sum in
//               float32, writes P = 2^(s*c - m*c) rounded to bfloat16 back over the first half
//               of S's columns (tcgen05.st), and at the item's end normalises and stores its row of O;
//   warp 4      one thread issues the MMAs: S = Q K^T (operands in shared memory, eight
//               tcgen05.mma of K 16), and O += P V with P read from tensor memory and V as an
//               MN-major operand straight from the page layout (keys along K);
//   warps 5-7   TMA producers: an item's query tile, then per tile of 128 keys the pages that the
//               block table names, each as two boxes of [page x 64] into 128-byte-swizzled
//               tiles, two stages each for K and V.  Two warps bring K, one brings V (a K tile is
//               never queued behind the wait for a V buffer); a warp issues the copies of its
//               lanes one after the other, so K's boxes are dealt out over lanes of both warps.
// The roles run ahead of one another across items: the producers load the next item's Q, K and V
// while the current one is computed (two Q buffers), and O has two buffers, so that the next item's
// products start while the softmax warps still write the last item's output.
// S has two buffers: S[j+1] is issued before O += P[j] V[j], so that it is complete when the
// softmax warps finish tile j, and the tensor core works on tile j+1 and on P[j] V[j] while they
// compute tile j+1's exponentials.
//
// The running maximum is only moved when a row's new maximum exceeds it by more than 2^8 in the
// exponent: P then stays below 256, which bfloat16 holds with the same relative rounding, and O
// (in tensor memory) is rescaled only then.  Sum and output use the same maximum, so the result
// is the exact softmax up to rounding.
//
// Keys above the diagonal, below the window or beyond the sequence are masked to -inf before the
// maximum is taken; pages that hold no visible key are not loaded.  What such a page's place in
// the V buffer holds must be finite (0 * NaN would poison the row): the buffer is zeroed at the
// start and afterwards only ever receives pages of the pool, which the engine allocates zeroed.
//
// Every wait is bounded by a clock limit; a role that gives up sets an error word that the host
// can read, the block lets its copies land, frees its tensor memory and returns.
//
// Role in the reference: pulsar-core/inc/pulsar/kernels/paged_prefill.cuh:35-346 (mma.sync tiles
// of 16 queries with a host-built tile list).
#include "attention_tcgen05.cuh"

#include <cstdlib>

namespace {

using namespace pb;
using namespace pb::attn5;

constexpr int kThreads = 256;             // 4 softmax warps, the MMA warp, 3 producer warps
constexpr int kKProducers = 2;           // warps that bring K; one more brings V
constexpr int kStages = 2;                     // K and V tiles in flight
constexpr int kSmemBytes = (2 + 2 * kStages) * kTileBytes + 1024 /* alignment slack */ + 256 /* barriers */;
constexpr int kTmemColumns = 512;              // S[0] | S[1] (P over the first 64 of each) | O[0] | O[1]

__device__ unsigned int g_attn5_error = 0;     // 0 = fine; else 1 + the role that gave up

// Barrier slots; those of K and V exist once per stage, those of Q, S, P and O once per buffer.
enum { kBarOFull = 0, kBarODone, kBarQFull, kBarQEmpty = kBarQFull + 2, kBarOEmpty = kBarQEmpty + 2, kBarSFull = kBarOEmpty + 2,
       kBarPFull = kBarSFull + 2, kBarKFull = kBarPFull + 2, kBarKEmpty = kBarKFull + kStages,
       kBarVFull = kBarKEmpty + kStages, kBarVEmpty = kBarVFull + kStages, kNumBars = kBarVEmpty + kStages };

struct Args {
    bf16* out;
    const int* block_table;
    const int* cu_q;
    const int* kv_len;
    int table_stride, n_seqs, n_items, Hq, Hkv, page_shift, rows_per_load, window;
    float scale;
    PoolBounds bounds;
};

// One work item: a tile of 128 query rows of one sequence and one query head.  Every role of a block
// walks the same list of items: item k of block b is number k*G + b (k even) or k*G + G-1-b (k odd) of
// the grid's G blocks, the items being numbered with the head fastest and the tiles backwards (longest
// key ranges first), so that each block gets about the same number of key tiles.
struct Work {
    int t;                     // items of this block so far
    int head, kvh, q_row0, rows, pos_first, pos_last, lo, kt0, n_tiles;
    const int* table;
};

__device__ __forceinline__ bool next_item(Work& w, const Args& a) {
    const int k = w.t;
    const int G = gridDim.x, b = blockIdx.x;
    const int idx = k * G + ((k & 1) ? G - 1 - b : b);
    if (idx >= a.n_items) return false;
    const int n_q_tiles = a.n_items / a.Hq;
    w.head = idx % a.Hq;
    w.kvh = w.head / (a.Hq / a.Hkv);
    int tile = n_q_tiles - 1 - idx / a.Hq;
    int s = 0, q0 = 0, q_len = 0;
    for (; s < a.n_seqs; ++s) {
        q0 = a.cu_q[s];
        q_len = a.cu_q[s + 1] - q0;
        const int nt = (q_len + kBM - 1) / kBM;
        if (tile < nt) break;
        tile -= nt;
    }
    if (s >= a.n_seqs) return false;                            // the caller's tile count does not match cu_q
    const int m0 = tile * kBM;
    w.rows = min(kBM, q_len - m0);
    w.q_row0 = q0 + m0;
    const int ctx0 = a.kv_len[s] - q_len;
    w.pos_first = ctx0 + m0;
    w.pos_last = ctx0 + m0 + w.rows - 1;
    w.lo = (a.window > 0 && w.pos_first - a.window + 1 > 0) ? w.pos_first - a.window + 1 : 0;
    w.kt0 = w.lo / kBN;
    w.n_tiles = w.pos_last / kBN - w.kt0 + 1;
    w.table = a.block_table + (size_t)s * a.table_stride;
    w.t = k + 1;
    return true;
}

__global__ void __launch_bounds__(kThreads, 1)
prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const Args a) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* q_s = smem;                                 // two tiles
    unsigned char* k_s = smem + 2 * kTileBytes;                // kStages tiles
    unsigned char* v_s = smem + (2 + kStages) * kTileBytes;    // kStages tiles
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (2 + 2 * kStages) * kTileBytes);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kNumBars);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t bar0 = smem_addr(bars);
    auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };

    // V's buffers start finite (see the header); 16 bytes per thread and step.
    for (int i = tid; i < kStages * kTileBytes / 16; i += kThreads) reinterpret_cast<uint4*>(v_s)[i] = make_uint4(0, 0, 0, 0);
    if (tid == 0) {
        for (int i = 0; i < kNumBars; ++i) {
            const bool from_softmax = (i >= kBarPFull && i < kBarPFull + 2) || (i >= kBarOEmpty && i < kBarOEmpty + 2);
            const bool from_k_producers = i >= kBarKFull && i < kBarKEmpty;
            mbar_init(bar(i), from_softmax ? 4 : from_k_producers ? kKProducers : 1);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // the zeros are visible to the TMA/MMA proxy
    if (warp == 4) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(kTmemColumns));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 2 * kBN;      // S[0] | S[1] | O[0] | O[1]

    if (warp >= 5) {
        // ---------------- TMA producers.  Warps 5 and 6 bring K (and warp 5 the query tiles), warp 7 brings V, so
        // that a K tile, which the next S product waits for, is never queued behind the wait for a V buffer.  A warp
        // issues the copies of its lanes one after the other, so a tile's boxes are dealt out over lanes of two warps.
        const bool for_v = warp == 7;
        const int pw = warp - 5;                               // K: 0 or 1
        const int loads = kBN / a.rows_per_load;               // pages (or parts of a page) per tile
        const uint32_t load_bytes = (uint32_t)a.rows_per_load * 128u;
        const int box = for_v ? lane : pw + kKProducers * lane;      // box -> (page slot, half)
        const int slot = box >> 1, half = box & 1;
        unsigned char* tiles = for_v ? v_s : k_s;
        const CUtensorMap* map = for_v ? &map_v : &map_k;
        const int bar_full = for_v ? kBarVFull : kBarKFull, bar_empty = for_v ? kBarVEmpty : kBarKEmpty;
        bool ok = true;
        uint32_t g = 0;                                        // key tiles so far, over all items
        Work w;
        w.t = 0;
        while (ok && next_item(w, a)) {
            const int t = w.t - 1, qb = t & 1;
            if (warp == 5) {
                if (lane == 0) {
                    ok = mbar_wait(bar(kBarQEmpty + qb), ((t >> 1) & 1) ^ 1, abort_flag);      // the item before last has used it
                    if (ok) {
                        const uint32_t dst = smem_addr(q_s) + (uint32_t)qb * kTileBytes;
                        mbar_expect_tx(bar(kBarQFull + qb), kTileBytes);
                        tma_load_2d(dst, &map_q, bar(kBarQFull + qb), w.head * kD, w.q_row0);
                        tma_load_2d(dst + kHalfBytes, &map_q, bar(kBarQFull + qb), w.head * kD + 64, w.q_row0);
                    }
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
            }
            for (int j = 0; j < w.n_tiles && ok; ++j, ++g) {
                const int key0 = (w.kt0 + j) * kBN;
                const int st = g % kStages;
                const uint32_t free_parity = ((g / kStages) & 1) ^ 1;
                const int key = key0 + slot * a.rows_per_load;
                const bool want = slot < loads && key + a.rows_per_load > w.lo && key <= w.pos_last;
                int row = 0;
                if (want) {
                    int page = w.table[key >> a.page_shift];
                    if (!page_ok(page, a.bounds)) page = 0;
                    row = ((page * a.Hkv + w.kvh) << a.page_shift) + (key & ((1 << a.page_shift) - 1));
                }
                const uint32_t n_want = __popc(__ballot_sync(0xffffffffu, want));
                const uint32_t dst_off = (uint32_t)st * kTileBytes + (uint32_t)half * kHalfBytes + (uint32_t)(slot * a.rows_per_load) * 128u;
                // the stage is free when the product that read it last has retired
                if (lane == 0) {
                    ok = mbar_wait(bar(bar_empty + st), free_parity, abort_flag);
                    if (ok) mbar_expect_tx(bar(bar_full + st), n_want * load_bytes);
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                if (want) tma_load_2d(smem_addr(tiles) + dst_off, map, bar(bar_full + st), half * 64, row);
            }
        }
        if (!ok && lane == 0) { *abort_flag = 1; atomicMax(&g_attn5_error, 2u); }
    } else if (warp == 4) {
        // ---------------- MMA issuer.  Two cursors walk the block's key tiles: S is issued one tile ahead of
        // O += P V (also across items), so that the next S is complete when the softmax warps finish a tile.
        // S of tile g+1 overwrites the columns that held S and P of tile g-1: O += P V of tile g-1 was issued
        // before it, and the MMAs of one thread run in the order of their issue.  The whole warp walks the loop
        // and waits on the barriers, one elected lane issues: with uniform control flow the descriptors live in
        // uniform registers, and the issuing stream is short enough to keep up with the tensor core (which takes
        // an MMA only when the one before it has started) although a softmax warp shares the scheduler.
        {
            const uint32_t tmem_s = __shfl_sync(0xffffffffu, tmem_base, 0), tmem_o = tmem_s + 2 * kBN;
            const uint64_t q_desc = desc_k_major(smem_addr(q_s)), k_desc = desc_k_major(smem_addr(k_s));
            const uint64_t v_desc = desc_mn_major(smem_addr(v_s));
            Work ws, wp;                                       // the items of the S cursor and of the P V cursor
            ws.t = wp.t = 0;
            int js = 0, jp = 0;                                // tile within the item
            uint32_t gs = 0, gp = 0;                           // tile over all items
            bool more_s = next_item(ws, a), more_p = next_item(wp, a);
            bool ok = true;
            auto issue_s = [&]() -> bool {
                const int t = ws.t - 1, qb = t & 1;
                const int st = gs % kStages, sb = gs & 1;
                if (js == 0 && !mbar_wait(bar(kBarQFull + qb), (t >> 1) & 1, abort_flag)) return false;
                if (!mbar_wait(bar(kBarKFull + st), (gs / kStages) & 1, abort_flag)) return false;
                fence_after();
                // descriptors differ from tile to tile only in their address field (16-byte units): a 64-bit add each
                const uint64_t qd = q_desc + (uint64_t)((uint32_t)qb * (kTileBytes >> 4));
                const uint64_t kd = k_desc + (uint64_t)((uint32_t)st * (kTileBytes >> 4));
                ++js;
                ++gs;
                const bool last = js == ws.n_tiles;
                if (elect_one()) {
#pragma unroll
                    for (int ks = 0; ks < kD / 16; ++ks) {
                        constexpr uint32_t kHalf16 = kHalfBytes >> 4;
                        const uint32_t off = (uint32_t)(ks >> 2) * kHalf16 + (uint32_t)(ks & 3) * 2u;      // 32 bytes per k-step
                        umma_ss(tmem_s + (uint32_t)sb * kBN, qd + off, kd + off, kIdescS, ks > 0 ? 1u : 0u);
                    }
                    umma_commit(bar(kBarKEmpty + st));
                    umma_commit(bar(kBarSFull + sb));
                    if (last) umma_commit(bar(kBarQEmpty + qb));     // the item's last S: its Q buffer is free once it has retired
                }
                __syncwarp();
                if (last) {
                    js = 0;
                    more_s = next_item(ws, a);
                }
                return true;
            };
            if (more_s) ok = issue_s();
            while (ok && more_p) {
                if (more_s && !issue_s()) { ok = false; break; }
                const int t = wp.t - 1, ob = t & 1;
                const int st = gp % kStages, sb = gp & 1;
                // the item before last has been read out of this O buffer
                if (jp == 0 && !mbar_wait(bar(kBarOEmpty + ob), ((t >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
                if (!mbar_wait(bar(kBarVFull + st), (gp / kStages) & 1, abort_flag)) { ok = false; break; }
                if (!mbar_wait(bar(kBarPFull + sb), (gp >> 1) & 1, abort_flag)) { ok = false; break; }
                fence_after();
                const uint64_t vd = v_desc + (uint64_t)((uint32_t)st * (kTileBytes >> 4));
                const bool item_done = jp + 1 == wp.n_tiles;
                if (elect_one()) {
#pragma unroll
                    for (int kk = 0; kk < kBN / 16; ++kk)
                        umma_ts(tmem_o + (uint32_t)ob * kD, tmem_s + (uint32_t)sb * kBN + (uint32_t)kk * 8u, vd + (uint64_t)(kk * (2048 >> 4)),
                                kIdescPV, (jp > 0 || kk > 0) ? 1u : 0u);
                    umma_commit(bar(kBarVEmpty + st));
                    umma_commit(bar(kBarOFull));
                    if (item_done) umma_commit(bar(kBarODone));      // the item's O is complete once everything issued so far has retired
                }
                __syncwarp();
                ++jp;
                ++gp;
                if (item_done) {
                    jp = 0;
                    more_p = next_item(wp, a);
                }
            }
            if (!ok && lane == 0) { *abort_flag = 1; atomicMax(&g_attn5_error, 3u); }
        }
    } else {
        // ---------------- softmax: thread `r` owns query row r
        const int r = warp * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
        const float sl2 = a.scale * kLog2e;
        const int window = a.window;
        bool ok = true;
        uint32_t g = 0;
        Work w;
        w.t = 0;
        while (ok && next_item(w, a)) {
            const int t = w.t - 1, ob = t & 1;
            const int pos = w.pos_first + min(r, w.rows - 1);     // rows beyond the tile's end repeat the last one
            const uint32_t tmem_ot = tmem_o + (uint32_t)ob * kD + lane_addr;
            float m_used = -INFINITY, l_run = 0.0f;
            for (int j = 0; j < w.n_tiles; ++j, ++g) {
                const int sb = g & 1;
                const uint32_t tmem_sj = tmem_s + (uint32_t)sb * kBN + lane_addr;
                ok = mbar_wait(bar(kBarSFull + sb), (g >> 1) & 1, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                fence_after();
                const int key0 = (w.kt0 + j) * kBN;
                // every row of the block sees every key of the tile?
                const bool all_visible = key0 + kBN - 1 <= w.pos_first && (window <= 0 || key0 > w.pos_last - window);
                // the whole row of S into registers: four loads in flight, one wait
                uint32_t v[kBN];
#pragma unroll
                for (int c = 0; c < kBN; c += 32) tmem_ld32_nowait(tmem_sj + c, *reinterpret_cast<uint32_t(*)[32]>(&v[c]));
                tmem_wait_ld();
#pragma unroll
                for (int c = 0; c < kBN; c += 32) tmem_landed(*reinterpret_cast<uint32_t(*)[32]>(&v[c]));
                if (!all_visible) {
                    // columns lo..hi of the tile are visible to this row; compared without branches
                    const int hi = pos - key0;
                    const int lo = window > 0 ? pos - window + 1 - key0 : -(1 << 30);
#pragma unroll
                    for (int i = 0; i < kBN; ++i) v[i] = ((i <= hi) & (i >= lo)) ? v[i] : __float_as_uint(-INFINITY);
                }
                float tm[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int i = 0; i < kBN; i += 4) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) tm[e] = fmaxf(tm[e], __uint_as_float(v[i + e]));
                }
                const float tmax = fmaxf(fmaxf(tm[0], tm[1]), fmaxf(tm[2], tm[3]));
                // move the maximum only when it grew by more than the lazy threshold
                float corr = 1.0f;
                if ((tmax - m_used) * sl2 > kLazyRescale) {      // also the first visible key: m_used = -inf
                    corr = ex2((m_used - tmax) * sl2);            // 0 when m_used = -inf
                    m_used = tmax;
                    l_run *= corr;
                }
                const float neg_ms = (m_used == -INFINITY) ? 0.0f : -m_used * sl2;
                // P over the first half of S's columns
                float l0 = 0.0f, l1 = 0.0f;
#pragma unroll
                for (int c = 0; c < kBN; c += 32) {
                    uint32_t p[16];
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float p0 = ex2(fmaf(__uint_as_float(v[c + i]), sl2, neg_ms));
                        const float p1 = ex2(fmaf(__uint_as_float(v[c + i + 1]), sl2, neg_ms));
                        l0 += p0;
                        l1 += p1;
                        p[i >> 1] = pack_bf16x2(p0, p1);
                    }
                    tmem_st16(tmem_sj + (c >> 1), p);
                }
                l_run += l0 + l1;
                if (j > 0 && __any_sync(0xffffffffu, corr != 1.0f)) {
                    // O is rescaled in place once O += P V of the tile before has retired (that of this tile waits
                    // for this warp's P)
                    ok = mbar_wait(bar(kBarOFull), (g - 1) & 1, abort_flag);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    fence_after();
#pragma unroll 1
                    for (int c = 0; c < kD; c += 32) {
                        uint32_t o[32];
                        tmem_ld32(tmem_ot + c, o);
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
                        tmem_st32(tmem_ot + c, o);
                    }
                }
                tmem_wait_st();
                fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(kBarPFull + sb));
            }
            if (!ok) break;
            // the item's output: O of its last tile has retired.  (A barrier of its own: a warp whose rows see nothing of
            // the last tiles gets here while kBarOFull is still two phases behind, which a parity cannot tell from none.)
            ok = mbar_wait(bar(kBarODone), t & 1, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            fence_after();
            const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
            bf16* dst = a.out + ((size_t)(w.q_row0 + r) * a.Hq + w.head) * kD;
#pragma unroll 1
            for (int c = 0; c < kD; c += 32) {
                uint32_t o[32];
                tmem_ld32(tmem_ot + c, o);
                if (r < w.rows) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        uint32_t x[4];
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            x[k] = pack_bf16x2(__uint_as_float(o[i * 8 + 2 * k]) * inv, __uint_as_float(o[i * 8 + 2 * k + 1]) * inv);
                        reinterpret_cast<uint4*>(dst + c)[i] = make_uint4(x[0], x[1], x[2], x[3]);
                    }
                }
            }
            fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(kBarOEmpty + ob));       // this warp's lanes of the O buffer may be overwritten
        }
        if (!ok && lane == 0) {
            *abort_flag = 1;
            atomicMax(&g_attn5_error, 4u);
        }
    }
    __syncwarp();
    if (*abort_flag) {
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);       // copies in flight land before the memory is reused
    }
    fence_before();
    __syncthreads();
    if (warp == 4) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemColumns));
}

// PULSAR_ATTENTION_HEADS=1 keeps one query head per block also where a group's heads could share a block.
int heads_per_block() {
    static int n = [] {
        const char* e = getenv("PULSAR_ATTENTION_HEADS");
        return (e && e[0] == '1' && e[1] == 0) ? 1 : 2;
    }();
    return n;
}

}  // namespace

// Query rows per block: the caller sizes the grid as the sum over sequences of ceil(q_len / this).
PB_EXPORT int pb_prefill_tcgen05_tile(void) { return kBM; }

PB_EXPORT int pb_prefill_tcgen05_supported(int dtype, int Hq, int Hkv, int D, int page_size) {
    if (dtype != PB_BF16 || Hkv <= 0 || Hq % Hkv) return 0;
    if (D != kD) return 0;
    if (log2_exact(page_size) < 0 || page_size < 8) return 0;           // whole groups of 8 swizzled rows per page
    return 1;
}

// The error word of the kernel's bounded waits (0 = no block ever gave up); reading it synchronises.
PB_EXPORT int pb_prefill_tcgen05_error(void) {
    unsigned int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_attn5_error, sizeof(v)) != cudaSuccess) return -1;
    const int dual = dual_error();
    if (dual < 0) return -1;
    return (int)v > dual ? (int)v : dual;
}

// As pb_gemm_tcgen05_wait_control, for the two attention kernels: ``addresses`` receives two device addresses
// (the one-head kernel's error word, the two-head kernel's).
PB_EXPORT int pb_prefill_tcgen05_wait_control(long long limit, int error, void** addresses) {
    if (wait_control(g_attn5_error, limit, error, addresses) != 0) return -1;
    return dual_wait_control(limit, error, addresses ? addresses + 1 : nullptr);
}

// q, out [N, Hq, D] bfloat16; pools [n_pages, Hkv, page_size, D] bfloat16 with finite contents;
// n_q_tiles = sum over sequences of ceil(q_len / pb_prefill_tcgen05_tile()).
PB_EXPORT int pb_paged_attention_prefill_tcgen05(int dtype, const void* q, const void* k_pool, const void* v_pool, void* out,
                                                 const int* block_table, int table_stride, const int* cu_q,
                                                 const int* kv_len, int n_tokens, int n_seqs, int n_q_tiles, int n_pages,
                                                 int Hq, int Hkv, int D, int page_size, float scale, int window,
                                                 cudaStream_t stream) {
    if (n_seqs <= 0 || n_q_tiles <= 0 || n_tokens <= 0) return 0;
    if (!pb_prefill_tcgen05_supported(dtype, Hq, Hkv, D, page_size)) return PB_ERR_BAD_SIZE;
    const long long items = (long long)n_q_tiles * Hq;
    if (items >= (1LL << 30)) return PB_ERR_TOO_LARGE;
    if ((((uintptr_t)q | (uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)out) & 15) != 0) return PB_ERR_BAD_SIZE;
    if (heads_per_block() == 2 && dual_supported(Hq, Hkv))
        return launch_dual(q, k_pool, v_pool, out, block_table, table_stride, cu_q, kv_len, n_tokens, n_seqs, n_q_tiles, n_pages, Hq,
                           Hkv, page_size, scale, window, stream);
    const long long pool_rows = (long long)n_pages * Hkv * page_size;
    if (pool_rows >= (1LL << 31)) return PB_ERR_TOO_LARGE;
    const int rows_per_load = page_size < kBN ? page_size : kBN;
    CUtensorMap mq, mk, mv;
    int rc = make_map(&mq, q, n_tokens, (long long)Hq * D, kBM);
    if (rc != 0) return rc;
    rc = make_map(&mk, k_pool, pool_rows, D, rows_per_load);
    if (rc != 0) return rc;
    rc = make_map(&mv, v_pool, pool_rows, D, rows_per_load);
    if (rc != 0) return rc;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(prefill_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    Args a;
    a.out = (bf16*)out;
    a.block_table = block_table;
    a.cu_q = cu_q;
    a.kv_len = kv_len;
    a.table_stride = table_stride;
    a.n_seqs = n_seqs;
    a.n_items = (int)items;
    a.Hq = Hq;
    a.Hkv = Hkv;
    a.page_shift = log2_exact(page_size);
    a.rows_per_load = rows_per_load;
    a.window = window;
    a.scale = scale;
    a.bounds = pool_bounds_now();
    const int grid = (int)(items < sm_count() ? items : sm_count());       // persistent: one block per SM
    prefill_tcgen05_kernel<<<grid, kThreads, kSmemBytes, stream>>>(mq, mk, mv, a);
    return launch_status();
}
