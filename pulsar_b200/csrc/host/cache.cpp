#include "cache.h"

#include <algorithm>

namespace ph {

FreeList::FreeList(int n) : n_(n), held_(n > 0 ? n : 0, 0) {
    free_.reserve(n > 0 ? n : 0);
    for (int i = n - 1; i >= 0; --i) free_.push_back(i);
}

int FreeList::take() {
    if (free_.empty()) return kOutOfPages;
    const int id = free_.back();
    free_.pop_back();
    held_[id] = 1;
    return id;
}

int FreeList::give(int id) {
    if (id < 0 || id >= n_ || !held_[id]) return kNotHeld;
    held_[id] = 0;
    free_.push_back(id);
    return 0;
}

Cache::Cache(int n_groups, const int* windows, const int* pages, int page_size, int max_requests)
    : page_size_(page_size), slots_(max_requests) {
    groups_.reserve(n_groups);
    for (int g = 0; g < n_groups; ++g) {
        groups_.push_back(Group{windows[g], FreeList(pages[g])});
        if (windows[g] > 0) windowed_ = true;
    }
}

const Request* Cache::find(int64_t rid) const {
    auto it = reqs_.find(rid);
    return it == reqs_.end() ? nullptr : &it->second;
}
Request* Cache::find(int64_t rid) {
    auto it = reqs_.find(rid);
    return it == reqs_.end() ? nullptr : &it->second;
}

int Cache::open(int64_t rid) {
    if (reqs_.count(rid)) return kAlreadyOpen;
    const int slot = slots_.take();
    if (slot < 0) return kOutOfSlots;
    Request r;
    r.slot = slot;
    r.tables.resize(groups_.size());
    r.released.assign(groups_.size(), 0);
    r.synced.assign(groups_.size(), 0);
    reqs_.emplace(rid, std::move(r));
    return slot;
}

void Cache::set_resident_tables(bool on) {
    resident_tables_ = on;
    for (auto& kv : reqs_) kv.second.synced.assign(groups_.size(), 0);      // nothing is known to be on the device
}

// Logical pages below this hold only keys that no query at position >= length sees.
int Cache::first_needed_page(const Group& g, int length) const {
    if (g.window <= 0) return 0;
    const int first_key = length - g.window + 1;          // oldest key the query at `length` sees
    return std::max(0, first_key) / page_size_;
}

int Cache::pages_to_append(const Request& r, int n_new, int group) const {
    const int have = (int)r.tables[group].size();
    const int need = (r.length + n_new + page_size_ - 1) / page_size_;
    return std::max(0, need - have);
}

int Cache::reclaimable(const Request& r, int group) const {
    const int upto = std::min(first_needed_page(groups_[group], r.length), (int)r.tables[group].size());
    return std::max(0, upto - r.released[group]);
}

bool Cache::can_append(const Request& r, int n_new) const {
    for (int g = 0; g < n_groups(); ++g)
        if (pages_to_append(r, n_new, g) > groups_[g].pages.n_free() + reclaimable(r, g)) return false;
    return true;
}

bool Cache::can_admit(int n_tokens) const {
    const int pages = (n_tokens + page_size_ - 1) / page_size_;
    if (slots_.n_free() <= 0) return false;
    for (const Group& g : groups_)
        if (pages > g.pages.n_free()) return false;
    return true;
}

int Cache::release_passed(Request& r) {
    if (!windowed_) return 0;
    int n = 0;
    for (int g = 0; g < n_groups(); ++g) {
        std::vector<int>& table = r.tables[g];
        const int upto = std::min(first_needed_page(groups_[g], r.length), (int)table.size());
        for (int lp = r.released[g]; lp < upto; ++lp) {
            if (groups_[g].pages.give(table[lp]) != 0) return kNotHeld;
            table[lp] = -1;
            ++n;
        }
        r.released[g] = std::max(r.released[g], upto);
    }
    return n;
}

int Cache::append(int64_t rid, int n_new) {
    if (n_new <= 0) return kBadArgument;
    Request* r = find(rid);
    if (!r) return kUnknownRequest;
    if (!can_append(*r, n_new)) return kOutOfPages;        // either every group gets its pages or nothing changes
    const int rc = release_passed(*r);
    if (rc < 0) return rc;
    for (int g = 0; g < n_groups(); ++g) {
        const int need = pages_to_append(*r, n_new, g);
        for (int i = 0; i < need; ++i) r->tables[g].push_back(groups_[g].pages.take());
    }
    const int start = r->length;
    r->length += n_new;
    return start;
}

int Cache::close(int64_t rid) {
    auto it = reqs_.find(rid);
    if (it == reqs_.end()) return kUnknownRequest;
    Request& r = it->second;
    int rc = 0;
    for (int g = 0; g < n_groups(); ++g)
        for (int page : r.tables[g])
            if (page >= 0 && groups_[g].pages.give(page) != 0) rc = kNotHeld;
    if (slots_.give(r.slot) != 0) rc = kNotHeld;
    reqs_.erase(it);
    return rc;
}

// Every page is free or held by exactly one request; every slot likewise.
int Cache::check() const {
    for (int g = 0; g < n_groups(); ++g) {
        std::vector<uint8_t> seen(groups_[g].pages.n(), 0);
        int count = 0;
        for (const auto& kv : reqs_)
            for (int page : kv.second.tables[g]) {
                if (page < 0) continue;
                if (page >= groups_[g].pages.n() || seen[page] || !groups_[g].pages.held(page)) return kInconsistent;
                seen[page] = 1;
                ++count;
            }
        if (count + groups_[g].pages.n_free() != groups_[g].pages.n()) return kInconsistent;      // a page was lost
    }
    std::vector<uint8_t> seen(slots_.n(), 0);
    int count = 0;
    for (const auto& kv : reqs_) {
        const int s = kv.second.slot;
        if (s < 0 || s >= slots_.n() || seen[s] || !slots_.held(s)) return kInconsistent;
        seen[s] = 1;
        ++count;
    }
    return count + slots_.n_free() == slots_.n() ? 0 : kInconsistent;
}

}  // namespace ph
