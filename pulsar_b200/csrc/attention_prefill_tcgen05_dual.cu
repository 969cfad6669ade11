// Paged prefill attention on the fifth-generation tensor cores, two query heads of one key/value group per block.
//
// Same work, layout and arithmetic as the one-head kernel beside it (causal, ragged batch, optional window, bfloat16
// pages, head size 128, lazily moved maximum), but a block takes a tile of 128 query tokens for TWO heads that share
// their keys and values.  Each K and V tile that comes from L2 then serves 256 query rows instead of 128: with one head
// per block every SM pulls 64 KB per key tile, which at full tensor rate would be twice what L2 delivers.  And the two
// heads' softmax warps (one warp of each per scheduler) alternate with the tensor core: while the warps of head A
// compute tile j's exponentials, it works on head B's products, and the other way round.
//
// Roles (384 threads):
//   warps 0-3   softmax of head A: thread r owns query row r (tensor-memory lane r) of S_A, P_A and O_A;
//   warps 4-7   the same for head B;
//   warps 8, 9  one thread of each issues one head's MMAs in the order  O += P[j] V[j],  S[j+1] = Q K[j+1]^T  (also
//               across items): a head has one S buffer, which P overwrites in part and the next S product reuses after
//               the P V product that read it (the MMAs of one thread run in the order of their issue).  Two issuing
//               threads, because the tensor core takes an MMA only when the one before has started: every barrier wait
//               of a lone issuing thread (some 60 cycles even when it passes at once) is time without products;
//   warps 10-11 TMA producers: 10 brings the two query tiles and K, 11 brings V.
// Tensor memory: S_A | S_B | O_A | O_B, 128 columns each.  Shared memory: Q_A, Q_B, two stages each of K and V.
// The softmax warps raise their register allowance (setmaxnreg), the others lower theirs.
//
// Every wait is bounded by a clock limit; a role that gives up sets an error word that the host can read, the block
// lets its copies land, frees its tensor memory and returns.
//
// Role in the reference: pulsar-core/inc/pulsar/kernels/paged_prefill.cuh:35-346.
#include "attention_tcgen05.cuh"

namespace {

using namespace pb;
using namespace pb::attn5;

constexpr int kThreads = 384;
constexpr int kSoftmaxWarps = 8;          // 4 per head
constexpr int kMmaWarp = 8;               // warps 8 and 9 issue the MMAs of head A and of head B
constexpr int kProducerWarp = 10;         // warp 10 brings Q and K, warp 11 brings V
constexpr int kStages = 2;
constexpr int kStageOutBytes = 4096;      // per softmax warp: 32 rows of 64 output columns
constexpr int kSmemBytes = (2 + 2 * kStages) * kTileBytes + 1024 /* alignment slack */ + 256 /* barriers */ + 1280 /* sequence bounds */ +
                           kSoftmaxWarps * kStageOutBytes;
static_assert(kSmemBytes <= 227 * 1024, "shared memory of one block");
constexpr int kTmemColumns = 512;
// Registers per thread: the block is launched with kRegsLaunch each (what 384 threads leave of the register file, in
// steps of 8); the four other warps give up what the eight softmax warps take.  setmaxnreg.inc waits, without a limit,
// until the registers it asks for are free, so the others must release at least as many.
constexpr int kRegsLaunch = 168, kRegsSoftmax = 200, kRegsOther = 104;
static_assert(128 * (kRegsLaunch - kRegsOther) >= 256 * (kRegsSoftmax - kRegsLaunch), "the softmax warps' registers must come from the others'");
static_assert(kRegsLaunch * kThreads <= 65536 && kRegsSoftmax % 8 == 0 && kRegsOther % 8 == 0, "register budget");

__device__ unsigned int g_dual_error = 0;      // 0 = fine; else 1 + the role that gave up

// Barrier slots; those of K and V exist once per stage, the others once per head.
enum { kBarQFull = 0, kBarQEmpty = 2, kBarSFull = 4, kBarPFull = 6, kBarPRest = 8, kBarOFull = 10, kBarODone = 12, kBarOEmpty = 14,
       kBarKFull = 16, kBarKEmpty = kBarKFull + kStages, kBarVFull = kBarKEmpty + kStages, kBarVEmpty = kBarVFull + kStages,
       kBarTurn = kBarVEmpty + kStages, kNumBars = kBarTurn + 2 };

// Half a row of P (64 keys) from the row of S in registers: 2^(s * sl2 + neg_ms) as bfloat16 pairs into 32 columns, the
// sums of the even and odd columns added to l0 and l1.
template <int kHalf>
__device__ __forceinline__ void store_p_half(const uint32_t (&v)[kBN], float sl2, float neg_ms, uint32_t tmem_sx, float& l0, float& l1) {
#pragma unroll
    for (int c = kHalf * (kBN / 2); c < (kHalf + 1) * (kBN / 2); c += 32) {
        uint32_t p[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
            const float p0 = ex2(fmaf(__uint_as_float(v[c + i]), sl2, neg_ms));
            const float p1 = ex2(fmaf(__uint_as_float(v[c + i + 1]), sl2, neg_ms));
            l0 += p0;
            l1 += p1;
            p[i >> 1] = pack_bf16x2(p0, p1);
        }
        tmem_st16(tmem_sx + (c >> 1), p);
    }
}

__device__ __forceinline__ float row_max(const uint32_t (&v)[kBN]) {
    float tm[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
    for (int i = 0; i < kBN; i += 4) {
#pragma unroll
        for (int e = 0; e < 4; ++e) tm[e] = fmaxf(tm[e], __uint_as_float(v[i + e]));
    }
    return fmaxf(fmaxf(tm[0], tm[1]), fmaxf(tm[2], tm[3]));
}

// The warp's stores to tensor memory are complete; one lane tells the issuing warp.
__device__ __forceinline__ void hand_over(uint32_t bar, int lane) {
    tmem_wait_st();
    fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(bar);
}

constexpr int kSeqCache = 128;           // sequences whose bounds a block keeps in shared memory

struct Args {
    bf16* out;
    const int* block_table;
    const int* cu_q;
    const int* kv_len;
    int table_stride, n_seqs, n_items, Hq, Hkv, page_shift, rows_per_load, window;
    int pairs, n_q_tiles, group;      // Hq / 2, n_items / pairs, Hq / Hkv
    float scale;
    PoolBounds bounds;
};

// One work item: a tile of 128 query rows of one sequence and a pair of query heads (2p, 2p+1) of one group.  Items are
// numbered with the pair fastest and the tiles backwards (longest key ranges first) and dealt out in snake order.
struct Work {
    int t;                     // items of this block so far
    int head, kvh, q_row0, rows, pos_first, pos_last, lo, kt0, n_tiles;
    const int* table;
};

// Where the sequences' bounds are read from: the block's copy in shared memory, or global memory for a large batch.
struct Seqs {
    const int* cu_q;
    const int* kv_len;
};

__device__ __forceinline__ bool next_item(Work& w, const Args& a, const Seqs& seqs) {
    const int k = w.t;
    const int G = gridDim.x, b = blockIdx.x;
    const int idx = k * G + ((k & 1) ? G - 1 - b : b);
    if (idx >= a.n_items) return false;
    const unsigned q_tile = (unsigned)idx / (unsigned)a.pairs;          // (one division per item: the counts come with the arguments)
    w.head = 2 * (idx - (int)q_tile * a.pairs);
    w.kvh = (int)((unsigned)w.head / (unsigned)a.group);
    int tile = a.n_q_tiles - 1 - (int)q_tile;
    int s = 0, q0 = 0, q_len = 0;
    for (; s < a.n_seqs; ++s) {
        q0 = seqs.cu_q[s];
        q_len = seqs.cu_q[s + 1] - q0;
        const int nt = (q_len + kBM - 1) / kBM;
        if (tile < nt) break;
        tile -= nt;
    }
    if (s >= a.n_seqs) return false;                            // the caller's tile count does not match cu_q
    const int m0 = tile * kBM;
    w.rows = min(kBM, q_len - m0);
    w.q_row0 = q0 + m0;
    const int ctx0 = seqs.kv_len[s] - q_len;
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
prefill_tcgen05_dual_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, const Args a) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* q_s = smem;                                 // Q_A, Q_B
    unsigned char* k_s = smem + 2 * kTileBytes;                // kStages tiles
    unsigned char* v_s = smem + (2 + kStages) * kTileBytes;    // kStages tiles
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (2 + 2 * kStages) * kTileBytes);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kNumBars);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* seq_s = reinterpret_cast<int*>(smem + (2 + 2 * kStages) * kTileBytes + 256);      // cu_q[0..n], then kv_len[0..n)
    unsigned char* out_s = smem + (2 + 2 * kStages) * kTileBytes + 256 + 1280;               // kStageOutBytes per softmax warp
    const bool cached = a.n_seqs <= kSeqCache;
    const Seqs seqs = {cached ? seq_s : a.cu_q, cached ? seq_s + kSeqCache + 1 : a.kv_len};

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t bar0 = smem_addr(bars);
    auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };

    // V's buffers start finite: a page that is not loaded leaves its place as it was, and 0 * NaN would poison a row.
    for (int i = tid; i < kStages * kTileBytes / 16; i += kThreads) reinterpret_cast<uint4*>(v_s)[i] = make_uint4(0, 0, 0, 0);
    if (cached) {
        // every role looks an item's sequence up in these bounds, once per item: from shared memory the walk over
        // the sequences costs a tenth of what dependent loads from global memory do
        for (int i = tid; i <= a.n_seqs; i += kThreads) seq_s[i] = a.cu_q[i];
        for (int i = tid; i < a.n_seqs; i += kThreads) seq_s[kSeqCache + 1 + i] = a.kv_len[i];
    }
    if (tid == 0) {
        for (int i = 0; i < kNumBars; ++i) {
            const bool from_softmax = (i >= kBarPFull && i < kBarPRest + 2) || (i >= kBarOEmpty && i < kBarOEmpty + 2);
            const bool from_both_issuers = (i >= kBarKEmpty && i < kBarKEmpty + kStages) || (i >= kBarVEmpty && i < kBarVEmpty + kStages);
            mbar_init(bar(i), from_softmax ? 4 : from_both_issuers ? 2 : 1);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // the zeros are visible to the TMA/MMA proxy
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(kTmemColumns));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 2 * kBN;      // S_A | S_B | O_A | O_B

    if (warp >= kSoftmaxWarps) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther));
        if (warp >= kProducerWarp) {
            // ---------------- TMA producers
            const bool for_v = warp == kProducerWarp + 1;
            const int pw = warp - kProducerWarp;
            const int loads = kBN / a.rows_per_load;               // pages (or parts of a page) per tile
            const uint32_t load_bytes = (uint32_t)a.rows_per_load * 128u;
            const int box = lane;                                  // box -> (page slot, half)
            const int slot = box >> 1, half = box & 1;
            unsigned char* tiles = for_v ? v_s : k_s;
            const CUtensorMap* map = for_v ? &map_v : &map_k;
            const int bar_full = for_v ? kBarVFull : kBarKFull, bar_empty = for_v ? kBarVEmpty : kBarKEmpty;
            bool ok = true;
            uint32_t g = 0;                                        // key tiles so far, over all items
            Work w;
            w.t = 0;
            while (ok && next_item(w, a, seqs)) {
                const int t = w.t - 1;
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
                    if (lane == 0) {
                        ok = mbar_wait(bar(bar_empty + st), free_parity, abort_flag);      // the products that read it last have retired
                        if (ok) mbar_expect_tx(bar(bar_full + st), n_want * load_bytes);
                    }
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (!ok) break;
                    if (want) tma_load_2d(smem_addr(tiles) + dst_off, map, bar(bar_full + st), half * 64, row);
                    if (j == 0 && pw == 0) {
                        // the item's query tiles, behind its first K tile: that one's buffer is free earlier than
                        // the query buffers, which the item before gives up with its last S products
                        if (lane == 0) {
                            for (int x = 0; x < 2 && ok; ++x) {
                                ok = mbar_wait(bar(kBarQEmpty + x), (t & 1) ^ 1, abort_flag);
                                if (ok) {
                                    const uint32_t dst = smem_addr(q_s) + (uint32_t)x * kTileBytes;
                                    mbar_expect_tx(bar(kBarQFull + x), kTileBytes);
                                    tma_load_2d(dst, &map_q, bar(kBarQFull + x), (w.head + x) * kD, w.q_row0);
                                    tma_load_2d(dst + kHalfBytes, &map_q, bar(kBarQFull + x), (w.head + x) * kD + 64, w.q_row0);
                                }
                            }
                        }
                        ok = __shfl_sync(0xffffffffu, ok, 0);
                    }
                }
            }
            if (!ok && lane == 0) { *abort_flag = 1; atomicMax(&g_dual_error, 2u); }
        } else {
            // ---------------- MMA issuers, one warp per head: while one of them waits for its head's P or for a tile,
            // the other's products keep the tensor core busy.  (A single thread that issues both heads' products
            // leaves it idle during every wait: an MMA is accepted only when the one before it has started.)  Per head
            // the order is  S[0],  then per tile  O += P[j] V[j],  S[j+1]  (also across items): the next S reuses the
            // columns that P[j] was read from, and the MMAs of one thread run in the order of their issue.  The whole
            // warp walks the loop and waits on the barriers, and one elected lane issues: with uniform control flow the
            // descriptors live in uniform registers, and the issuing stream is short enough to keep up with the tensor
            // core although the scheduler is shared with two softmax warps.
            const int x = __shfl_sync(0xffffffffu, warp, 0) - kMmaWarp;       // (a broadcast: the compiler sees it as uniform)
            const uint32_t tmem_s = __shfl_sync(0xffffffffu, tmem_base, 0), tmem_o = tmem_s + 2 * kBN;
            const uint64_t q_desc = desc_k_major(smem_addr(q_s)) + (uint64_t)((uint32_t)x * (kTileBytes >> 4));
            const uint64_t k_desc = desc_k_major(smem_addr(k_s));
            const uint64_t v_desc = desc_mn_major(smem_addr(v_s));
            const uint32_t tmem_sx = tmem_s + (uint32_t)x * kBN, tmem_ox = tmem_o + (uint32_t)x * kD;
            Work ws, wp;                                       // the items of the S cursor and of the P V cursor
            ws.t = wp.t = 0;
            int js = 0, jp = 0;                                // tile within the item
            uint32_t gs = 0, gp = 0;                           // tile over all items
            uint32_t turn = 0;                                 // this thread's turns so far
            bool more_s = next_item(ws, a, seqs), more_p = next_item(wp, a, seqs);
            bool ok = true;
            // The two threads take turns (A, B, A, ...), a turn being O += P[j] V[j] and S[j+1] of the thread's head, so
            // that one head's products run while the other head's softmax warps work; left alone, both heads fall into
            // step and softmax and products no longer overlap.  A thread does all its waiting before it asks for its
            // turn, and hands the turn on as soon as its MMAs are issued.
            auto begin_turn = [&]() -> bool {
                if (x == 0) return turn == 0 || mbar_wait(bar(kBarTurn + 0), (turn - 1) & 1, abort_flag);
                return mbar_wait(bar(kBarTurn + 1), turn & 1, abort_flag);
            };
            auto end_turn = [&]() {
                if (elect_one()) mbar_arrive(bar(kBarTurn + (x ^ 1)));
                __syncwarp();
                ++turn;
            };
            auto wait_s = [&]() -> bool {                      // Q and K of the S cursor's tile are there
                const int t = ws.t - 1;
                if (js == 0 && !mbar_wait(bar(kBarQFull + x), t & 1, abort_flag)) return false;
                return mbar_wait(bar(kBarKFull + gs % kStages), (gs / kStages) & 1, abort_flag);
            };
            auto issue_s = [&]() {
                const int st = gs % kStages;
                const uint64_t kd = k_desc + (uint64_t)((uint32_t)st * (kTileBytes >> 4));
                ++js;
                ++gs;
                const bool last = js == ws.n_tiles;
                if (elect_one()) {
#pragma unroll
                    for (int ks = 0; ks < kD / 16; ++ks) {
                        constexpr uint32_t kHalf16 = kHalfBytes >> 4;
                        const uint32_t off = (uint32_t)(ks >> 2) * kHalf16 + (uint32_t)(ks & 3) * 2u;      // 32 bytes per k-step
                        umma_ss(tmem_sx, q_desc + off, kd + off, kIdescS, ks > 0 ? 1u : 0u);
                    }
                    umma_commit(bar(kBarSFull + x));
                    umma_commit(bar(kBarKEmpty + st));         // free once both heads' products have read it
                    if (last) umma_commit(bar(kBarQEmpty + x));      // the item's last S of this head: its Q may go
                }
                __syncwarp();
                if (last) {
                    js = 0;
                    more_s = next_item(ws, a, seqs);
                }
            };
            if (more_s) {
                ok = wait_s() && begin_turn();
                if (ok) {
                    fence_after();
                    issue_s();
                    end_turn();
                }
            }
            while (ok && more_p) {
                const int t = wp.t - 1;
                const int st = gp % kStages;
                // the item before has been read out of this O buffer
                if (jp == 0 && !mbar_wait(bar(kBarOEmpty + x), (t & 1) ^ 1, abort_flag)) { ok = false; break; }
                if (!mbar_wait(bar(kBarVFull + st), (gp / kStages) & 1, abort_flag)) { ok = false; break; }
                if (more_s && !wait_s()) { ok = false; break; }
                if (!mbar_wait(bar(kBarPFull + x), gp & 1, abort_flag)) { ok = false; break; }
                if (!begin_turn()) { ok = false; break; }
                fence_after();
                const uint64_t vd = v_desc + (uint64_t)((uint32_t)st * (kTileBytes >> 4));
                const bool item_done = jp + 1 == wp.n_tiles;
                // the first half of P's columns (64 keys) is there: their products run while the softmax warps finish the rest
                if (elect_one()) {
#pragma unroll
                    for (int kk = 0; kk < kBN / 32; ++kk)
                        umma_ts(tmem_ox, tmem_sx + (uint32_t)kk * 8u, vd + (uint64_t)(kk * (2048 >> 4)), kIdescPV, (jp > 0 || kk > 0) ? 1u : 0u);
                }
                __syncwarp();
                if (!mbar_wait(bar(kBarPRest + x), gp & 1, abort_flag)) { ok = false; break; }
                fence_after();
                if (elect_one()) {
#pragma unroll
                    for (int kk = kBN / 32; kk < kBN / 16; ++kk)
                        umma_ts(tmem_ox, tmem_sx + (uint32_t)kk * 8u, vd + (uint64_t)(kk * (2048 >> 4)), kIdescPV, 1u);
                    umma_commit(bar(kBarOFull + x));
                    umma_commit(bar(kBarVEmpty + st));
                    if (item_done) umma_commit(bar(kBarODone + x));       // the item's O of this head is complete
                }
                __syncwarp();
                ++jp;
                ++gp;
                if (more_s) issue_s();
                end_turn();
                if (item_done) {
                    jp = 0;
                    more_p = next_item(wp, a, seqs);
                }
            }
            if (!ok && lane == 0) { *abort_flag = 1; atomicMax(&g_dual_error, 3u); }
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));
        // ---------------- softmax: thread `r` of head x owns query row r
        const int x = warp >> 2, wr = warp & 3;
        const int r = wr * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(wr * 32) << 16;
        const uint32_t tmem_sx = tmem_s + (uint32_t)x * kBN + lane_addr;
        const uint32_t tmem_ox = tmem_o + (uint32_t)x * kD + lane_addr;
        const float sl2 = a.scale * kLog2e;
        const int window = a.window;
        bool ok = true;
        uint32_t g = 0;
        Work w;
        w.t = 0;
        while (ok && next_item(w, a, seqs)) {
            const int t = w.t - 1;
            const int pos = w.pos_first + min(r, w.rows - 1);     // rows beyond the tile's end repeat the last one
            float m_used = -INFINITY, l_run = 0.0f;
            for (int j = 0; j < w.n_tiles; ++j, ++g) {
                ok = mbar_wait(bar(kBarSFull + x), g & 1, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                fence_after();
                const int key0 = (w.kt0 + j) * kBN;
                // every row of the block sees every key of the tile?
                const bool all_visible = key0 + kBN - 1 <= w.pos_first && (window <= 0 || key0 > w.pos_last - window);
                // the whole row of S into registers: four loads in flight, one wait
                uint32_t v[kBN];
#pragma unroll
                for (int c = 0; c < kBN; c += 32) tmem_ld32_nowait(tmem_sx + c, *reinterpret_cast<uint32_t(*)[32]>(&v[c]));
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
                const float tmax = row_max(v);
                // move the maximum only when it grew by more than the lazy threshold
                float corr = 1.0f;
                if ((tmax - m_used) * sl2 > kLazyRescale) {      // also the first visible key: m_used = -inf
                    corr = ex2((m_used - tmax) * sl2);            // 0 when m_used = -inf
                    m_used = tmax;
                    l_run *= corr;
                }
                if (j > 0 && __any_sync(0xffffffffu, corr != 1.0f)) {
                    // O is rescaled in place, before any product of this tile adds to it: O += P V of the tile before
                    // has retired (this tile's S was issued after it)
                    ok = mbar_wait(bar(kBarOFull + x), (g - 1) & 1, abort_flag);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    fence_after();
#pragma unroll 1
                    for (int c = 0; c < kD; c += 32) {
                        uint32_t o[32];
                        tmem_ld32(tmem_ox + c, o);
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
                        tmem_st32(tmem_ox + c, o);
                    }
                }
                // P lies over the first half of S's columns and is handed over in two halves of 64 keys
                const float neg_ms = (m_used == -INFINITY) ? 0.0f : -m_used * sl2;
                float l0 = 0.0f, l1 = 0.0f;
                store_p_half<0>(v, sl2, neg_ms, tmem_sx, l0, l1);
                hand_over(bar(kBarPFull + x), lane);
                store_p_half<1>(v, sl2, neg_ms, tmem_sx, l0, l1);
                hand_over(bar(kBarPRest + x), lane);
                l_run += l0 + l1;
            }
            if (!ok) break;
            // the item's output: O of its last tile has retired.  (A barrier of its own: a warp whose rows see nothing of
            // the last tiles gets here while kBarOFull is still phases behind, which a parity cannot tell from none.)
            ok = mbar_wait(bar(kBarODone + x), t & 1, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            fence_after();
            const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
            // the whole row of O into registers, so that the next item's products may overwrite the buffer while
            // the row is still being normalised and written
            uint32_t o[kD];
#pragma unroll
            for (int c = 0; c < kD; c += 32) tmem_ld32_nowait(tmem_ox + c, *reinterpret_cast<uint32_t(*)[32]>(&o[c]));
            tmem_wait_ld();
#pragma unroll
            for (int c = 0; c < kD; c += 32) tmem_landed(*reinterpret_cast<uint32_t(*)[32]>(&o[c]));
            fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(kBarOEmpty + x));       // this warp's lanes of the O buffer may be overwritten
            // The rows go out through shared memory, 64 columns at a time: a thread holds a whole row, and 32 threads
            // storing 16 bytes each to 32 rows make 32 memory transactions per instruction, which hold up the SM's
            // load/store pipe (and every barrier poll behind them) for thousands of cycles per item.  Transposed, a
            // store instruction writes four rows of 128 contiguous bytes.  16-byte chunk c of row q lies at chunk
            // c ^ (q & 7) of the row's 128 bytes, so that neither the writes nor the reads conflict.
            uint4* mine = reinterpret_cast<uint4*>(out_s + warp * kStageOutBytes);
            bf16* base = a.out + ((size_t)(w.q_row0 + wr * 32) * a.Hq + w.head + x) * kD;
            const int rows_here = w.rows - wr * 32;               // rows of this warp inside the tile
#pragma unroll
            for (int h = 0; h < 2; ++h) {
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    uint32_t y[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        y[k] = pack_bf16x2(__uint_as_float(o[h * 64 + c * 8 + 2 * k]) * inv, __uint_as_float(o[h * 64 + c * 8 + 2 * k + 1]) * inv);
                    mine[lane * 8 + (c ^ (lane & 7))] = make_uint4(y[0], y[1], y[2], y[3]);
                }
                __syncwarp();
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const int q = k * 4 + (lane >> 3), c = lane & 7;
                    const uint4 val = mine[q * 8 + (c ^ (q & 7))];
                    if (q < rows_here) *reinterpret_cast<uint4*>(base + (size_t)q * a.Hq * kD + h * 64 + c * 8) = val;
                }
                __syncwarp();
            }
        }
        if (!ok && lane == 0) {
            *abort_flag = 1;
            atomicMax(&g_dual_error, 4u);
        }
    }
    __syncwarp();
    if (*abort_flag) {
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);       // copies in flight land before the memory is reused
    }
    fence_before();
    __syncthreads();
    if (warp == kMmaWarp) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemColumns));
}

}  // namespace

namespace pb {
namespace attn5 {

// The register hand-over inside the kernel is sized for the count the kernel was compiled to; with another count
// setmaxnreg.inc could wait for ever, so the kernel is then not used.
static bool registers_as_planned() {
    static bool fine = [] {
        cudaFuncAttributes at;
        if (cudaFuncGetAttributes(&at, prefill_tcgen05_dual_kernel) != cudaSuccess) return false;
        const int regs = (at.numRegs + 7) / 8 * 8;
        return regs <= kRegsLaunch && 128 * (regs - kRegsOther) >= 256 * (kRegsSoftmax - regs);
    }();
    return fine;
}

bool dual_supported(int Hq, int Hkv) { return Hkv > 0 && Hq % Hkv == 0 && (Hq / Hkv) % 2 == 0 && registers_as_planned(); }

int dual_error() {
    unsigned int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_dual_error, sizeof(v)) != cudaSuccess) return -1;
    return (int)v;
}

int dual_wait_control(long long limit, int error, void** address) { return wait_control(g_dual_error, limit, error, address); }

// Arguments as those of the one-head launch; n_q_tiles counts tiles of 128 query rows.
int launch_dual(const void* q, const void* k_pool, const void* v_pool, void* out, const int* block_table, int table_stride,
                const int* cu_q, const int* kv_len, int n_tokens, int n_seqs, int n_q_tiles, int n_pages, int Hq, int Hkv,
                int page_size, float scale, int window, cudaStream_t stream) {
    const long long items = (long long)n_q_tiles * (Hq / 2);
    if (items >= (1LL << 30)) return PB_ERR_TOO_LARGE;
    const long long pool_rows = (long long)n_pages * Hkv * page_size;
    if (pool_rows >= (1LL << 31)) return PB_ERR_TOO_LARGE;
    const int rows_per_load = page_size < kBN ? page_size : kBN;
    CUtensorMap mq, mk, mv;
    int rc = make_map(&mq, q, n_tokens, (long long)Hq * kD, kBM);
    if (rc != 0) return rc;
    rc = make_map(&mk, k_pool, pool_rows, kD, rows_per_load);
    if (rc != 0) return rc;
    rc = make_map(&mv, v_pool, pool_rows, kD, rows_per_load);
    if (rc != 0) return rc;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(prefill_tcgen05_dual_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
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
    a.pairs = Hq / 2;
    a.n_q_tiles = n_q_tiles;
    a.group = Hq / Hkv;
    a.page_shift = log2_exact(page_size);
    a.rows_per_load = rows_per_load;
    a.window = window;
    a.scale = scale;
    a.bounds = pool_bounds_now();
    const int grid = (int)(items < sm_count() ? items : sm_count());       // persistent: one block per SM
    prefill_tcgen05_dual_kernel<<<grid, kThreads, kSmemBytes, stream>>>(mq, mk, mv, a);
    return launch_status();
}

}  // namespace attn5
}  // namespace pb
