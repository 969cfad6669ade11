// Continuous batching above the step function: admission, prompt portions under a token budget,
// decoding, finishing, and what happens when pages run out.
//
// Order of one step, as in the reference (pulsar-core/src/runtime/scheduler.cpp:76-222): first
// every running request that is past its prompt gets one decode token, then prompts in progress
// continue in running order, then waiting requests are admitted first-in first-out, the head of
// the queue blocking those behind it.  Decisions that differ from the reference:
//   * the budget counts every token of the step, decoded ones included (the reference counts
//     prompt tokens only, scheduler.cpp:100);
//   * admission looks at the whole prompt plus one token, not at the first portion
//     (scheduler.cpp:154-170), and the pages a running prompt still needs are held back from later
//     admissions, so two half-fed prompts can never starve each other;
//   * when a decoding request cannot get its next page the request admitted last is preempted: its
//     pages go back, it returns to the head of the queue and is recomputed from its tokens later
//     (the reference throws "out of pages": pulsar-core/src/runtime/kv/active_buffer.cpp:153-160);
//   * when nothing at all can run because pages are held by requests that wait for a further turn on kept
//     pages (or by a prompt in progress beside them), the holder furthest back in the queue gives its pages up
//     and is recomputed; if no waiting request holds any, the running request admitted last is preempted;
//   * a request that could never fit the pool alone is refused when it is submitted.
// A step may be decided while the tokens of the step before are still on the device: such a token
// stands in the request's token list as kUnread until on_token fills it in.
#pragma once

#include "cache.h"

#include <deque>

namespace ph {

constexpr int kUnread = -1;

enum : int {
    kNeverFits = -20,
    kStillRunning = -21,
    kHasUnread = -22,
    kNoUnread = -23,
    kNeedsPreemption = -24,
};

struct Sequence {
    std::vector<int> tokens;
    int max_new_tokens = 0;
    int n_cached = 0;
    int n_generated = 0;
    long admitted_at = -1;      // admission counter value; larger = admitted later
    int preemptions = 0;
    int unread = 0;             // trailing tokens that are still kUnread
    bool spent = false;         // the turn's budget is used up: nothing more is scheduled for it
    int pending() const { return (int)tokens.size() - n_cached; }
};

struct PlanEntry {
    int64_t rid;
    int first;                  // index of the entry's first token in the request's token list
    int count;
    bool sample;                // the portion completes what the request knows: its last logits are wanted
};

class Scheduler {
public:
    Scheduler(Cache* cache, int max_running, int max_chunk_size);

    int add_request(int64_t rid, const int* tokens, int n, int max_new_tokens);
    int extend_request(int64_t rid, const int* tokens, int n, int max_new_tokens);
    bool has_work() const { return !waiting_.empty() || !running_.empty(); }
    int schedule(bool allow_preempt, std::vector<PlanEntry>* out);      // 0, or kNeedsPreemption
    void on_step(const std::vector<PlanEntry>& plan);
    int on_sampled(int64_t rid);
    int on_token(int64_t rid, int token, int eos_id);                    // 1 when the turn is over, 0 otherwise
    int drop_unread(int64_t rid);
    void park(int64_t rid);
    void finish(int64_t rid);

    const Sequence* find(int64_t rid) const;
    const std::deque<int64_t>& waiting() const { return waiting_; }
    const std::vector<int64_t>& running() const { return running_; }
    int n_preemptions() const { return n_preemptions_; }
    int max_running() const { return max_running_; }
    const std::vector<PlanEntry>& last_plan() const { return plan_; }
    std::vector<PlanEntry>& plan_buffer() { return plan_; }

private:
    int pages(int n_tokens) const { return (n_tokens + cache_->page_size() - 1) / cache_->page_size(); }
    int capacity_pages() const;
    int free_pages() const;
    int held_back() const;
    int pages_for(int64_t rid, int n_new) const;
    void preempt(int64_t rid);
    int plan_once(bool allow_preempt, std::vector<PlanEntry>* out);
    bool is_running(int64_t rid) const;

    Cache* cache_;
    int max_running_, max_chunk_size_;
    std::deque<int64_t> waiting_;
    std::vector<int64_t> running_;
    std::unordered_map<int64_t, Sequence> seqs_;
    long admissions_ = 0;
    int n_preemptions_ = 0;
    std::vector<PlanEntry> plan_;
};

}  // namespace ph
