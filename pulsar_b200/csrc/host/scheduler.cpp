#include "scheduler.h"

#include <algorithm>
#include <climits>

namespace ph {

Scheduler::Scheduler(Cache* cache, int max_running, int max_chunk_size)
    : cache_(cache), max_running_(std::min(max_running, cache->slots().n())), max_chunk_size_(max_chunk_size) {}

int Scheduler::capacity_pages() const {
    int n = INT_MAX;
    for (int g = 0; g < cache_->n_groups(); ++g) n = std::min(n, cache_->group(g).pages.n());
    return cache_->n_groups() ? n : (1 << 30);
}

int Scheduler::free_pages() const {
    int n = INT_MAX;
    for (int g = 0; g < cache_->n_groups(); ++g) n = std::min(n, cache_->group(g).pages.n_free());
    return cache_->n_groups() ? n : (1 << 30);
}

// Pages that running prompts still need to reach their last known token plus one.
int Scheduler::held_back() const {
    int total = 0;
    for (int64_t rid : running_) {
        const Sequence& s = seqs_.at(rid);
        total += std::max(0, pages((int)s.tokens.size() + 1) - pages(s.n_cached));
    }
    return total;
}

bool Scheduler::is_running(int64_t rid) const { return std::find(running_.begin(), running_.end(), rid) != running_.end(); }

const Sequence* Scheduler::find(int64_t rid) const {
    auto it = seqs_.find(rid);
    return it == seqs_.end() ? nullptr : &it->second;
}

int Scheduler::add_request(int64_t rid, const int* tokens, int n, int max_new_tokens) {
    if (seqs_.count(rid)) return kAlreadyOpen;
    if (n <= 0) return kBadArgument;
    if (pages(n + std::max(0, max_new_tokens)) > capacity_pages()) return kNeverFits;
    Sequence s;
    s.tokens.assign(tokens, tokens + n);
    s.max_new_tokens = max_new_tokens;
    seqs_.emplace(rid, std::move(s));
    waiting_.push_back(rid);
    return 0;
}

// More tokens for a known request that is not running (a further turn): it keeps its pages and
// waits for admission again.
int Scheduler::extend_request(int64_t rid, const int* tokens, int n, int max_new_tokens) {
    auto it = seqs_.find(rid);
    if (it == seqs_.end()) return kUnknownRequest;
    if (is_running(rid)) return kStillRunning;
    Sequence& s = it->second;
    if (n < 0) return kBadArgument;
    if (pages((int)s.tokens.size() + n + std::max(0, max_new_tokens)) > capacity_pages()) return kNeverFits;
    if (s.unread) return kHasUnread;
    // Nothing new and nothing left over to run (every token is cached already, as after a pass that ran one step
    // ahead and cached a stop token): a step could not bring a single token, so the request is not queued.
    if (n == 0 && (int)s.tokens.size() - s.n_cached <= 0) return kBadArgument;
    s.tokens.insert(s.tokens.end(), tokens, tokens + n);
    s.max_new_tokens = max_new_tokens;
    s.n_generated = 0;
    s.spent = false;
    if (std::find(waiting_.begin(), waiting_.end(), rid) == waiting_.end()) waiting_.push_back(rid);
    return 0;
}

void Scheduler::preempt(int64_t rid) {
    Sequence& s = seqs_.at(rid);
    if (cache_->has(rid)) cache_->close(rid);
    s.n_cached = 0;
    ++s.preemptions;
    ++n_preemptions_;
    running_.erase(std::find(running_.begin(), running_.end(), rid));
    waiting_.push_front(rid);
}

// Pages to reach the new length, beyond the logical pages the request already has.
int Scheduler::pages_for(int64_t rid, int n_new) const {
    const Request* r = cache_->find(rid);
    if (r && cache_->n_groups()) {
        int logical = INT_MAX;
        for (const auto& t : r->tables) logical = std::min(logical, (int)t.size());
        return std::max(0, pages(r->length + n_new) - logical);
    }
    return pages(n_new);
}

// Decides the next step.  Changes nothing in the cache except by preemption; the step packer takes the
// pages when it runs the entries.  With allow_preempt false (a step is still in flight, so some tokens are
// unread and nothing may be recomputed from them) the answer is kNeedsPreemption where a request would
// have to be preempted.
int Scheduler::schedule(bool allow_preempt, std::vector<PlanEntry>* out_ptr) {
    // When nothing at all can run although there is work, pages are held by requests that the three steps of
    // plan_once cannot touch: requests that wait for a further turn on kept pages, or a prompt in progress beside
    // them.  Then the holder furthest back in the queue gives its pages up (it is recomputed later); if no waiting
    // request holds any, the running request admitted last is preempted; and the step is decided again.
    for (;;) {
        const int rc = plan_once(allow_preempt, out_ptr);
        if (rc < 0 || !out_ptr->empty() || !allow_preempt || !has_work()) return rc;
        int64_t victim = -1;
        for (auto it = waiting_.rbegin(); it != waiting_.rend(); ++it)
            if (cache_->has(*it)) { victim = *it; break; }
        if (victim >= 0) {
            if (waiting_.size() == 1 && running_.empty()) return rc;        // it waits alone: its own pages do not block it
            Sequence& v = seqs_.at(victim);
            cache_->close(victim);
            v.n_cached = 0;
            ++v.preemptions;
            ++n_preemptions_;
            continue;
        }
        if (running_.size() + waiting_.size() < 2) return rc;             // one request alone that cannot run: the engine reports it
        if (running_.empty()) return rc;
        int64_t youngest = running_.front();
        for (int64_t r : running_)
            if (seqs_.at(r).admitted_at > seqs_.at(youngest).admitted_at) youngest = r;
        if (!cache_->has(youngest)) return rc;
        preempt(youngest);
    }
}

int Scheduler::plan_once(bool allow_preempt, std::vector<PlanEntry>* out_ptr) {
    std::vector<PlanEntry>& out = *out_ptr;
    out.clear();
    int budget = max_chunk_size_;
    int planned_pages = 0;                 // pages this step's entries will take
    const int ps = cache_->page_size();
    auto planned = [&](int64_t rid) {
        for (const PlanEntry& e : out)
            if (e.rid == rid) return true;
        return false;
    };

    // 1. decode tokens, oldest admission first; preempt the youngest when pages run out.
    std::vector<int64_t> decoders;
    for (int64_t rid : running_) {
        const Sequence& s = seqs_.at(rid);
        if (s.pending() == 1 && s.n_cached > 0 && !s.spent) decoders.push_back(rid);
    }
    std::stable_sort(decoders.begin(), decoders.end(),
                     [&](int64_t a, int64_t b) { return seqs_.at(a).admitted_at < seqs_.at(b).admitted_at; });
    for (int64_t rid : decoders) {
        if (!is_running(rid)) continue;            // preempted below
        if (budget <= 0) break;
        while (pages_for(rid, 1) > free_pages() - planned_pages) {
            if (!allow_preempt) return kNeedsPreemption;
            int64_t victim = running_.front();
            for (int64_t r : running_)
                if (seqs_.at(r).admitted_at > seqs_.at(victim).admitted_at) victim = r;
            for (size_t i = 0; i < out.size();) {   // its planned entry (and pages) leave the step
                if (out[i].rid == victim) {
                    budget += out[i].count;
                    planned_pages -= pages_for(victim, out[i].count);
                    out.erase(out.begin() + i);
                } else {
                    ++i;
                }
            }
            preempt(victim);
            if (victim == rid) break;
        }
        if (!is_running(rid)) continue;
        const Sequence& s = seqs_.at(rid);
        out.push_back(PlanEntry{rid, (int)s.tokens.size() - 1, 1, true});
        planned_pages += pages_for(rid, 1);
        budget -= 1;
    }

    // 2. prompts in progress, in running order.
    const std::vector<int64_t> in_order(running_);
    for (int64_t rid : in_order) {
        const Sequence& s = seqs_.at(rid);
        if (budget <= 0) break;
        if (planned(rid) || s.pending() == 0 || s.spent) continue;
        if (s.pending() == 1 && s.n_cached > 0) continue;          // a decoder that found no budget above
        // most new tokens that the free pages allow in this step (pages are held back for it, so it rarely shrinks)
        const int avail = std::max(0, free_pages() - planned_pages);
        const Request* r = cache_->find(rid);
        const int in_last = r ? ((ps - r->length % ps) % ps) : 0;
        const int n = std::min(std::min(s.pending(), budget), avail * ps + in_last);
        if (n <= 0) continue;
        out.push_back(PlanEntry{rid, s.n_cached, n, n == s.pending()});
        planned_pages += pages_for(rid, n);
        budget -= n;
    }

    // 3. admission, first-in first-out.
    while (!waiting_.empty() && (int)running_.size() < max_running_ && budget > 0) {
        const int64_t rid = waiting_.front();
        Sequence& s = seqs_.at(rid);
        const int have = cache_->has(rid) ? pages(s.n_cached) : 0;
        const int need_all = pages((int)s.tokens.size() + 1) - have;
        // what running requests still need (this step's pages included) stays theirs
        if (need_all > free_pages() - held_back()) break;           // head of the queue waits; nobody overtakes it
        if (!cache_->has(rid)) {
            int fresh = 0;
            for (const PlanEntry& e : out)
                if (!cache_->has(e.rid)) ++fresh;
            if (cache_->slots().n_free() - fresh <= 0) break;
        }
        waiting_.pop_front();
        running_.push_back(rid);
        s.admitted_at = admissions_++;
        const int n = std::min(s.pending(), budget);
        if (n <= 0) continue;                      // admitted with nothing to run (never queued so by extend_request)
        out.push_back(PlanEntry{rid, s.n_cached, n, n == s.pending()});
        planned_pages += pages_for(rid, n);
        budget -= n;
    }
    return 0;
}

void Scheduler::on_step(const std::vector<PlanEntry>& plan) {
    for (const PlanEntry& e : plan) {
        auto it = seqs_.find(e.rid);
        if (it != seqs_.end()) it->second.n_cached += e.count;      // a request that was finished meanwhile is gone
    }
}

// A token was sampled for the request on the device and is not read yet.
int Scheduler::on_sampled(int64_t rid) {
    auto it = seqs_.find(rid);
    if (it == seqs_.end()) return kUnknownRequest;
    Sequence& s = it->second;
    s.tokens.push_back(kUnread);
    ++s.unread;
    ++s.n_generated;
    if (s.n_generated >= s.max_new_tokens) s.spent = true;
    return 0;
}

// The oldest unread token has arrived (or, if none was announced, a token was sampled and read at once).
// 1 when the request's turn is over: stop token or budget (pulsar-core/src/runtime/engine.cpp:727-729).
int Scheduler::on_token(int64_t rid, int token, int eos_id) {
    auto it = seqs_.find(rid);
    if (it == seqs_.end()) return kUnknownRequest;
    Sequence& s = it->second;
    if (s.unread == 0) on_sampled(rid);
    s.tokens[s.tokens.size() - s.unread] = token;
    --s.unread;
    const bool spent_by_now = s.n_generated - s.unread >= s.max_new_tokens;
    return ((eos_id >= 0 && token == eos_id) || spent_by_now) ? 1 : 0;
}

// The newest unread token is void: the request had ended with the token before it.  (The step that sampled
// it has cached that last token, which is all it leaves.)
int Scheduler::drop_unread(int64_t rid) {
    auto it = seqs_.find(rid);
    if (it == seqs_.end()) return kUnknownRequest;
    Sequence& s = it->second;
    if (s.unread <= 0 || s.tokens.back() != kUnread) return kNoUnread;
    s.tokens.pop_back();
    --s.unread;
    --s.n_generated;
    return 0;
}

// The turn is over; the request leaves the running set and keeps its pages.
void Scheduler::park(int64_t rid) {
    auto it = std::find(running_.begin(), running_.end(), rid);
    if (it != running_.end()) running_.erase(it);
}

// Forget the request and give back what it holds.
void Scheduler::finish(int64_t rid) {
    park(rid);
    auto w = std::find(waiting_.begin(), waiting_.end(), rid);
    if (w != waiting_.end()) waiting_.erase(w);
    if (cache_->has(rid)) cache_->close(rid);
    seqs_.erase(rid);
}

}  // namespace ph
