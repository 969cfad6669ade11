// C interface of the host runtime (loaded with ctypes): the cache accounting of cache.h and the
// step packer, which grows the requests of a step in the cache and writes the step's index
// arrays into one (pinned) buffer that travels to the device in a single copy.
//
// The reference builds its per-step descriptor in Scheduler::step and Engine::build_prefill /
// build_decode with a host-to-device copy per array (pulsar-core/src/runtime/scheduler.cpp:58-72,
// 128-133, 172-220; pulsar-core/src/runtime/engine.cpp:573-702).
#include "cache.h"

#include <algorithm>
#include <cstring>

#define PH_EXPORT extern "C" __attribute__((visibility("default")))

using namespace ph;

namespace {
inline int align4(int n) { return (n + 3) / 4 * 4; }
}  // namespace

// ------------------------------------------------------------------ a free list of its own
PH_EXPORT void* ph_freelist_new(int n) { return n >= 0 ? new FreeList(n) : nullptr; }
PH_EXPORT void ph_freelist_delete(void* h) { delete static_cast<FreeList*>(h); }
PH_EXPORT int ph_freelist_take(void* h) { return static_cast<FreeList*>(h)->take(); }
PH_EXPORT int ph_freelist_give(void* h, int id) { return static_cast<FreeList*>(h)->give(id); }
PH_EXPORT int ph_freelist_n(void* h) { return static_cast<FreeList*>(h)->n(); }
PH_EXPORT int ph_freelist_n_free(void* h) { return static_cast<FreeList*>(h)->n_free(); }
PH_EXPORT int ph_freelist_held(void* h, int id) { return static_cast<FreeList*>(h)->held(id) ? 1 : 0; }

// ------------------------------------------------------------------ the cache
PH_EXPORT void* ph_cache_new(int n_groups, const int* windows, const int* pages, int page_size, int max_requests) {
    if (n_groups < 0 || page_size <= 0 || max_requests < 0) return nullptr;
    for (int g = 0; g < n_groups; ++g)
        if (pages[g] <= 0) return nullptr;
    return new Cache(n_groups, windows, pages, page_size, max_requests);
}
PH_EXPORT void ph_cache_delete(void* h) { delete static_cast<Cache*>(h); }
PH_EXPORT int ph_open(void* h, int64_t rid) { return static_cast<Cache*>(h)->open(rid); }
PH_EXPORT int ph_has(void* h, int64_t rid) { return static_cast<Cache*>(h)->has(rid) ? 1 : 0; }
PH_EXPORT int ph_length(void* h, int64_t rid) {
    const Request* r = static_cast<Cache*>(h)->find(rid);
    return r ? r->length : kUnknownRequest;
}
PH_EXPORT int ph_state_slot(void* h, int64_t rid) {
    const Request* r = static_cast<Cache*>(h)->find(rid);
    return r ? r->slot : kUnknownRequest;
}
// Logical pages the request's tables cover (the fewest over the groups).
PH_EXPORT int ph_n_logical_pages(void* h, int64_t rid) {
    const Request* r = static_cast<Cache*>(h)->find(rid);
    if (!r) return kUnknownRequest;
    int n = r->tables.empty() ? 0 : (int)r->tables[0].size();
    for (const auto& t : r->tables) n = std::min(n, (int)t.size());
    return n;
}
PH_EXPORT int ph_pages_to_append(void* h, int64_t rid, int n_new, int* out) {
    const Cache* c = static_cast<Cache*>(h);
    const Request* r = c->find(rid);
    if (!r) return kUnknownRequest;
    for (int g = 0; g < c->n_groups(); ++g) out[g] = c->pages_to_append(*r, n_new, g);
    return 0;
}
PH_EXPORT int ph_reclaimable(void* h, int64_t rid, int* out) {
    const Cache* c = static_cast<Cache*>(h);
    const Request* r = c->find(rid);
    if (!r) return kUnknownRequest;
    for (int g = 0; g < c->n_groups(); ++g) out[g] = c->reclaimable(*r, g);
    return 0;
}
PH_EXPORT int ph_can_append(void* h, int64_t rid, int n_new) {
    const Cache* c = static_cast<Cache*>(h);
    const Request* r = c->find(rid);
    if (!r) return kUnknownRequest;
    return c->can_append(*r, n_new) ? 1 : 0;
}
PH_EXPORT int ph_can_admit(void* h, int n_tokens) { return static_cast<Cache*>(h)->can_admit(n_tokens) ? 1 : 0; }
PH_EXPORT int ph_release_passed(void* h, int64_t rid) {
    Cache* c = static_cast<Cache*>(h);
    Request* r = c->find(rid);
    return r ? c->release_passed(*r) : kUnknownRequest;
}
PH_EXPORT int ph_append(void* h, int64_t rid, int n_new) { return static_cast<Cache*>(h)->append(rid, n_new); }
PH_EXPORT int ph_close(void* h, int64_t rid) { return static_cast<Cache*>(h)->close(rid); }
PH_EXPORT int ph_check(void* h) { return static_cast<Cache*>(h)->check(); }
PH_EXPORT int ph_n_free_pages(void* h, int group) { return static_cast<Cache*>(h)->group(group).pages.n_free(); }
PH_EXPORT int ph_n_pages(void* h, int group) { return static_cast<Cache*>(h)->group(group).pages.n(); }
PH_EXPORT int ph_page_held(void* h, int group, int page) { return static_cast<Cache*>(h)->group(group).pages.held(page) ? 1 : 0; }
PH_EXPORT int ph_n_free_slots(void* h) { return static_cast<Cache*>(h)->slots().n_free(); }
PH_EXPORT int ph_slot_held(void* h, int slot) { return static_cast<Cache*>(h)->slots().held(slot) ? 1 : 0; }
// The request's block table of one group: its length; the first min(length, cap) entries go to out.
PH_EXPORT int ph_table(void* h, int64_t rid, int group, int* out, int cap) {
    const Request* r = static_cast<Cache*>(h)->find(rid);
    if (!r) return kUnknownRequest;
    const std::vector<int>& t = r->tables[group];
    std::memcpy(out, t.data(), sizeof(int) * std::min((int)t.size(), cap));
    return (int)t.size();
}
// slot = page * page_size + offset for positions [start, start + n).
PH_EXPORT int ph_slots(void* h, int64_t rid, int group, int start, int n, int* out) {
    const Cache* c = static_cast<Cache*>(h);
    const Request* r = c->find(rid);
    if (!r) return kUnknownRequest;
    const std::vector<int>& t = r->tables[group];
    const int ps = c->page_size();
    if (start < 0 || n < 0 || (start + n + ps - 1) / ps > (int)t.size()) return kBadArgument;
    for (int p = start; p < start + n; ++p) {
        const int page = t[p / ps];
        if (page < 0) return kReleasedPage;
        out[p - start] = page * ps + p % ps;
    }
    return 0;
}

// ------------------------------------------------------------------ the step packer
// Entries i < n_entries: request rids[i] gets its next n_tok[i] tokens (concatenated in `tokens`); want_n[i]
// indices among them (concatenated in `wants`) name the rows whose logits are asked for; token_src[i] >= 0
// says that the entry's one token is element token_src[i] of the ids the step before sampled on the device.
//
// Phase 1 (ph_step_plan): checks the entries, gives back pages that windows have passed, checks that the
// whole step's pages and slots are there (nothing else changes if they are not: kOutOfPages / kOutOfSlots),
// then opens and grows the requests.  Fills starts[i] (position of the entry's first token), slots[i] (state
// slot) and widths[g] (block-table width of the step, rounded up to table_bucket for a step of single tokens)
// and returns the number of 32-bit words the packed buffer needs.  bad_entry gets the offending entry on error.
//
// Phase 2 (ph_step_pack): writes the arrays, each padded to 16 bytes, into `buf`:
//   token_ids, positions, seq_of_token [N]; cu_q [S+1]; kv_len, state_slots [S]; logit_rows [R];
//   per group: slots [N], block table [S, width] (-1 where a request has no page);
//   if any entry takes its token from the device: move_dst, move_src [number of such entries].
// With resident tables (ph_set_resident_tables) the device keeps a block-table row per state slot, and the per-group
// table array is replaced by the page ids the step's requests gained since they were last sent:
//   updates [1 + 3 * capacity]: the count, then (state slot, logical page, page id) triples; the capacity is the
//   number of entries for a step of single tokens (a token adds one page at most; the array's length then does not
//   change from step to step), else the exact count.  Packing marks those pages as sent.
// offsets/lengths receive where each array starts and how long it is (7 + 2 * groups (+ 2) entries).
namespace {
// Page ids of group g that the entries' requests hold and the device's resident table does not yet.
int unsynced_pages(const Cache& c, int g, int n_entries, const int64_t* rids) {
    int n = 0;
    for (int i = 0; i < n_entries; ++i) {
        const Request* r = c.find(rids[i]);
        n += std::max(0, (int)r->tables[g].size() - r->synced[g]);
    }
    return n;
}
int update_capacity(const Cache& c, int g, int n_entries, const int64_t* rids, bool all_single) {
    const int exact = unsynced_pages(c, g, n_entries, rids);
    return all_single ? std::max(exact, n_entries) : exact;
}
}  // namespace

PH_EXPORT void ph_set_resident_tables(void* h, int on) { static_cast<Cache*>(h)->set_resident_tables(on != 0); }

PH_EXPORT int ph_step_plan(void* h, int n_entries, const int64_t* rids, const int* n_tok, const int* tokens, const int* want_n,
                           const int* wants, const int* token_src, int n_sampled, int vocab, int table_bucket, int* starts,
                           int* slots, int* widths, int* bad_entry) {
    Cache* c = static_cast<Cache*>(h);
    const int G = c->n_groups(), ps = c->page_size();
    *bad_entry = -1;
    if (n_entries <= 0) return kBadArgument;
    int tok_at = 0, want_at = 0, fresh = 0;
    bool all_single = true;
    for (int i = 0; i < n_entries; ++i) {
        *bad_entry = i;
        if (n_tok[i] <= 0) return kBadArgument;
        for (int j = 0; j < i; ++j)
            if (rids[j] == rids[i]) return kAlreadyOpen;            // a request twice in one step
        for (int k = 0; k < n_tok[i]; ++k)
            if (tokens[tok_at + k] < 0 || tokens[tok_at + k] >= vocab) return kBadArgument;
        for (int k = 0; k < want_n[i]; ++k)
            if (wants[want_at + k] < 0 || wants[want_at + k] >= n_tok[i]) return kBadArgument;
        if (token_src[i] >= 0 && (n_tok[i] != 1 || token_src[i] >= n_sampled)) return kBadArgument;
        if (n_tok[i] != 1) all_single = false;
        if (!c->has(rids[i])) ++fresh;
        tok_at += n_tok[i];
        want_at += want_n[i];
    }
    *bad_entry = -1;
    if (fresh > c->slots().n_free()) return kOutOfSlots;
    // pages of the whole step before any request grows (pages that windows have passed serve this very step)
    std::vector<int> need(G, 0);
    for (int i = 0; i < n_entries; ++i) {
        Request* r = c->find(rids[i]);
        if (r) {
            const int rc = c->release_passed(*r);
            if (rc < 0) return rc;
            for (int g = 0; g < G; ++g) need[g] += c->pages_to_append(*r, n_tok[i], g);
        } else {
            for (int g = 0; g < G; ++g) need[g] += (n_tok[i] + ps - 1) / ps;
        }
    }
    for (int g = 0; g < G; ++g)
        if (need[g] > c->group(g).pages.n_free()) return kOutOfPages;
    for (int i = 0; i < n_entries; ++i) {
        if (!c->has(rids[i])) {
            const int rc = c->open(rids[i]);
            if (rc < 0) return rc;
        }
        starts[i] = c->append(rids[i], n_tok[i]);
        if (starts[i] < 0) { *bad_entry = i; return starts[i]; }
        slots[i] = c->find(rids[i])->slot;
    }
    int n = 0, rows = 0, moved = 0;
    for (int i = 0; i < n_entries; ++i) {
        n += n_tok[i];
        rows += want_n[i];
        if (token_src[i] >= 0) ++moved;
    }
    int total = 3 * align4(std::max(n, 1)) + align4(n_entries + 1) + 2 * align4(n_entries) + align4(std::max(rows, 1));
    for (int g = 0; g < G; ++g) {
        int w = 1;
        for (int i = 0; i < n_entries; ++i) w = std::max(w, (int)c->find(rids[i])->tables[g].size());
        if (all_single && table_bucket > 0) w = (w + table_bucket - 1) / table_bucket * table_bucket;
        widths[g] = w;
        const int table_words = c->resident_tables() ? 1 + 3 * update_capacity(*c, g, n_entries, rids, all_single) : n_entries * w;
        total += align4(std::max(n, 1)) + align4(table_words);
    }
    if (moved) total += 2 * align4(moved);
    return total;
}

PH_EXPORT int ph_step_pack(void* h, int n_entries, const int64_t* rids, const int* n_tok, const int* tokens, const int* want_n,
                           const int* wants, const int* token_src, const int* starts, const int* slots, const int* widths,
                           int* buf, int capacity, int* offsets, int* lengths) {
    Cache* c = static_cast<Cache*>(h);
    const int G = c->n_groups(), ps = c->page_size(), S = n_entries;
    int n = 0, rows = 0, moved = 0;
    bool all_single = true;
    for (int i = 0; i < S; ++i) {
        n += n_tok[i];
        rows += want_n[i];
        if (token_src[i] >= 0) ++moved;
        if (n_tok[i] != 1) all_single = false;
    }
    const bool resident = c->resident_tables();
    int k = 0, total = 0;
    auto place = [&](int len) {
        offsets[k] = total;
        lengths[k] = len;
        ++k;
        total += align4(std::max(len, 1));
    };
    place(n); place(n); place(n); place(S + 1); place(S); place(S); place(rows);
    for (int g = 0; g < G; ++g) {
        place(n);
        place(resident ? 1 + 3 * update_capacity(*c, g, S, rids, all_single) : S * widths[g]);
    }
    if (moved) { place(moved); place(moved); }
    if (total > capacity) return kTooSmall;
    int* tok = buf + offsets[0];
    int* pos = buf + offsets[1];
    int* seq = buf + offsets[2];
    int* cu = buf + offsets[3];
    int* kv = buf + offsets[4];
    int* slot = buf + offsets[5];
    int* lrow = buf + offsets[6];
    int at = 0, row_at = 0, tok_at = 0, want_at = 0, move_at = 0;
    cu[0] = 0;
    for (int i = 0; i < S; ++i) {
        const int q = n_tok[i];
        for (int j = 0; j < q; ++j) {
            tok[at + j] = tokens[tok_at + j];
            pos[at + j] = starts[i] + j;
            seq[at + j] = i;
        }
        for (int j = 0; j < want_n[i]; ++j) lrow[row_at++] = at + wants[want_at + j];
        if (token_src[i] >= 0) {
            buf[offsets[7 + 2 * G] + move_at] = at;
            buf[offsets[8 + 2 * G] + move_at] = token_src[i];
            ++move_at;
        }
        kv[i] = starts[i] + q;
        slot[i] = slots[i];
        at += q;
        tok_at += q;
        want_at += want_n[i];
        cu[i + 1] = at;
    }
    for (int g = 0; g < G; ++g) {
        int* sl = buf + offsets[7 + 2 * g];
        int* table = buf + offsets[8 + 2 * g];
        const int w = widths[g];
        if (resident) std::fill(table, table + lengths[8 + 2 * g], 0);
        else std::fill(table, table + (size_t)S * w, -1);
        at = 0;
        int n_upd = 0;
        for (int i = 0; i < S; ++i) {
            Request* r = c->find(rids[i]);
            const std::vector<int>& t = r->tables[g];
            for (int j = 0; j < n_tok[i]; ++j) {
                const int p = starts[i] + j;
                const int page = t[p / ps];
                if (page < 0) return kReleasedPage;
                sl[at + j] = page * ps + p % ps;
            }
            if (resident) {
                for (int lp = r->synced[g]; lp < (int)t.size(); ++lp) {
                    int* triple = table + 1 + 3 * n_upd++;
                    triple[0] = r->slot;
                    triple[1] = lp;
                    triple[2] = t[lp];
                }
            } else {
                std::memcpy(table + (size_t)i * w, t.data(), sizeof(int) * t.size());
            }
            at += n_tok[i];
        }
        if (resident) table[0] = n_upd;
    }
    if (resident)           // only now, with every array written: these pages count as sent
        for (int g = 0; g < G; ++g)
            for (int i = 0; i < S; ++i) {
                Request* r = c->find(rids[i]);
                r->synced[g] = (int)r->tables[g].size();
            }
    return total;
}

// ------------------------------------------------------------------ the scheduler
#include "scheduler.h"

PH_EXPORT void* ph_sched_new(void* cache, int max_running, int max_chunk_size) {
    if (!cache || max_running <= 0 || max_chunk_size <= 0) return nullptr;
    return new Scheduler(static_cast<Cache*>(cache), max_running, max_chunk_size);
}
PH_EXPORT void ph_sched_delete(void* h) { delete static_cast<Scheduler*>(h); }
PH_EXPORT int ph_sched_add(void* h, int64_t rid, const int* tokens, int n, int max_new_tokens) {
    return static_cast<Scheduler*>(h)->add_request(rid, tokens, n, max_new_tokens);
}
PH_EXPORT int ph_sched_extend(void* h, int64_t rid, const int* tokens, int n, int max_new_tokens) {
    return static_cast<Scheduler*>(h)->extend_request(rid, tokens, n, max_new_tokens);
}
PH_EXPORT int ph_sched_has_work(void* h) { return static_cast<Scheduler*>(h)->has_work() ? 1 : 0; }
// Decides a step and keeps it; returns the number of its entries, or kNeedsPreemption.
PH_EXPORT int ph_sched_schedule(void* h, int allow_preempt) {
    Scheduler* s = static_cast<Scheduler*>(h);
    const int rc = s->schedule(allow_preempt != 0, &s->plan_buffer());
    return rc < 0 ? rc : (int)s->last_plan().size();
}
// The step decided last: per entry the request, the index of its first token, the count and whether its last
// logits are wanted; returns the total number of tokens.
PH_EXPORT int ph_sched_plan(void* h, int64_t* rids, int* first, int* count, int* sample) {
    const Scheduler* s = static_cast<Scheduler*>(h);
    int total = 0, i = 0;
    for (const PlanEntry& e : s->last_plan()) {
        rids[i] = e.rid;
        first[i] = e.first;
        count[i] = e.count;
        sample[i] = e.sample ? 1 : 0;
        total += e.count;
        ++i;
    }
    return total;
}
// The tokens of the step decided last, entry after entry.
PH_EXPORT int ph_sched_plan_tokens(void* h, int* out) {
    const Scheduler* s = static_cast<Scheduler*>(h);
    int at = 0;
    for (const PlanEntry& e : s->last_plan()) {
        const Sequence* q = s->find(e.rid);
        if (!q) return kUnknownRequest;
        std::memcpy(out + at, q->tokens.data() + e.first, sizeof(int) * e.count);
        at += e.count;
    }
    return at;
}
// The entries of the step decided last ran: their tokens are cached now.
PH_EXPORT void ph_sched_on_step(void* h) {
    Scheduler* s = static_cast<Scheduler*>(h);
    s->on_step(s->last_plan());
}
PH_EXPORT int ph_sched_on_sampled(void* h, int64_t rid) { return static_cast<Scheduler*>(h)->on_sampled(rid); }
PH_EXPORT int ph_sched_on_token(void* h, int64_t rid, int token, int eos_id) {
    return static_cast<Scheduler*>(h)->on_token(rid, token, eos_id);
}
PH_EXPORT int ph_sched_drop_unread(void* h, int64_t rid) { return static_cast<Scheduler*>(h)->drop_unread(rid); }
PH_EXPORT void ph_sched_park(void* h, int64_t rid) { static_cast<Scheduler*>(h)->park(rid); }
PH_EXPORT void ph_sched_finish(void* h, int64_t rid) { static_cast<Scheduler*>(h)->finish(rid); }
PH_EXPORT int ph_sched_knows(void* h, int64_t rid) { return static_cast<Scheduler*>(h)->find(rid) ? 1 : 0; }
// info: n_tokens, max_new_tokens, n_cached, n_generated, admitted_at, preemptions, unread, spent.
PH_EXPORT int ph_sched_info(void* h, int64_t rid, int64_t* info) {
    const Sequence* q = static_cast<Scheduler*>(h)->find(rid);
    if (!q) return kUnknownRequest;
    info[0] = (int64_t)q->tokens.size();
    info[1] = q->max_new_tokens;
    info[2] = q->n_cached;
    info[3] = q->n_generated;
    info[4] = q->admitted_at;
    info[5] = q->preemptions;
    info[6] = q->unread;
    info[7] = q->spent ? 1 : 0;
    return 0;
}
PH_EXPORT int ph_sched_tokens(void* h, int64_t rid, int* out, int cap) {
    const Sequence* q = static_cast<Scheduler*>(h)->find(rid);
    if (!q) return kUnknownRequest;
    std::memcpy(out, q->tokens.data(), sizeof(int) * std::min((int)q->tokens.size(), cap));
    return (int)q->tokens.size();
}
PH_EXPORT int ph_sched_n_preemptions(void* h) { return static_cast<Scheduler*>(h)->n_preemptions(); }
PH_EXPORT int ph_sched_max_running(void* h) { return static_cast<Scheduler*>(h)->max_running(); }
// which: 0 = waiting (in order), 1 = running (in order); returns the count, fills min(count, cap).
PH_EXPORT int ph_sched_list(void* h, int which, int64_t* out, int cap) {
    const Scheduler* s = static_cast<Scheduler*>(h);
    int n = 0;
    if (which == 0) {
        for (int64_t r : s->waiting()) { if (n < cap) out[n] = r; ++n; }
    } else {
        for (int64_t r : s->running()) { if (n < cap) out[n] = r; ++n; }
    }
    return n;
}
