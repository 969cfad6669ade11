// Host-side accounting of the paged cache: page pools with LIFO free lists, one block table per
// request and group of layers, early release behind attention windows, state slots.  Plain C++
// (no CUDA): the device only ever sees the block tables and slot indices that the step packer
// (ph_step_pack in api.cpp) writes into a pinned buffer.
//
// What the reference's ActiveBuffer does for its one kind of layer
// (pulsar-core/src/runtime/kv/active_buffer.cpp:32-82 pools and free list, :152-228
// claim/allocate/append/free, :255-279 slot mapping) for several groups of layers.
#pragma once

#include <cstdint>
#include <unordered_map>
#include <vector>

namespace ph {

// Status codes of every entry point (>= 0 is success or a value).
enum : int {
    kUnknownRequest = -1,
    kAlreadyOpen = -2,
    kOutOfPages = -3,
    kOutOfSlots = -4,
    kBadArgument = -5,
    kReleasedPage = -6,
    kNotHeld = -7,
    kInconsistent = -8,
    kTooSmall = -9,
};

// LIFO free list over n ids: a fresh one yields 0, 1, 2, ...; a released id is the next one handed out.
class FreeList {
public:
    explicit FreeList(int n = 0);
    int n() const { return n_; }
    int n_free() const { return (int)free_.size(); }
    int take();                 // id, or kOutOfPages
    int give(int id);           // 0, or kNotHeld (freed twice, never taken, out of range)
    bool held(int id) const { return id >= 0 && id < n_ && held_[id]; }

private:
    int n_;
    std::vector<int> free_;
    std::vector<uint8_t> held_;
};

struct Group {
    int window;                 // keys a query sees at most; <= 0: all of them
    FreeList pages;
};

struct Request {
    int length = 0;
    int slot = -1;
    std::vector<std::vector<int>> tables;     // per group: logical page -> page id, or -1 once released
    std::vector<int> released;                // per group: logical pages [0, released) were given back
    std::vector<int> synced;                  // per group: logical pages [0, synced) are in the device's resident table
};

class Cache {
public:
    Cache(int n_groups, const int* windows, const int* pages, int page_size, int max_requests);

    int open(int64_t rid);                                      // state slot
    bool has(int64_t rid) const { return reqs_.count(rid) != 0; }
    const Request* find(int64_t rid) const;
    Request* find(int64_t rid);
    int pages_to_append(const Request& r, int n_new, int group) const;
    int reclaimable(const Request& r, int group) const;
    bool can_append(const Request& r, int n_new) const;
    bool can_admit(int n_tokens) const;
    int release_passed(Request& r);
    int append(int64_t rid, int n_new);                         // position of the first new token
    int close(int64_t rid);
    int check() const;                                          // 0 or kInconsistent

    int page_size() const { return page_size_; }
    int n_groups() const { return (int)groups_.size(); }
    const Group& group(int g) const { return groups_[g]; }
    const FreeList& slots() const { return slots_; }
    const std::unordered_map<int64_t, Request>& requests() const { return reqs_; }
    bool windowed() const { return windowed_; }
    // Resident tables: the device keeps one block-table row per state slot, and a step sends only the page ids that
    // its requests gained since they were last sent (see ph_step_pack).
    bool resident_tables() const { return resident_tables_; }
    void set_resident_tables(bool on);

private:
    int first_needed_page(const Group& g, int length) const;

    int page_size_;
    std::vector<Group> groups_;
    FreeList slots_;
    std::unordered_map<int64_t, Request> reqs_;
    bool windowed_ = false;
    bool resident_tables_ = false;
};

}  // namespace ph
