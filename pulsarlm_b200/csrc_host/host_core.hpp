// Host-side core of the engine in C++: the page pools and per-request block tables
// of the cache manager, and the scheduler's decisions. No CUDA here: the Python
// layer owns the tensors and the model; it asks this library which pages a request
// holds and which requests run next. Exposed through a C interface (host_core.cpp)
// and loaded with ctypes.
//
// The reference keeps the same concerns in C++: line_allocator / kv_cache
// (pulsarlm-core/src/engine/line_allocator.cpp, kv_cache.cpp) and scheduler /
// executor bookkeeping (src/engine/scheduler.cpp:36-109, executor.cpp:750-884).
#pragma once

#include <cstdint>
#include <deque>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

namespace plh {

// Page ids of one pool: taken all-or-nothing, given back once, reused last-in
// first-out (page 0 is taken first from a fresh pool).
class PagePool {
public:
    explicit PagePool(int n_pages);
    int n_pages() const { return static_cast<int>(held_.size()); }
    int free_count() const { return static_cast<int>(free_.size()); }
    int used_count() const { return n_pages() - free_count(); }
    int high_water() const { return high_water_; }
    bool is_held(int page) const { return page >= 0 && page < n_pages() && held_[page]; }
    // Appends `count` pages to `out`; false (nothing taken) when fewer are free.
    bool take(int count, std::vector<int>& out);
    // False (and nothing more given back) at the first page that is not held.
    bool give(const int* pages, int count);

private:
    std::vector<int> free_;   // stack: back() is taken next
    std::vector<char> held_;
    int high_water_ = 0;
};

enum Code : int {
    kOk = 0,
    kNoRoom = 1,          // too few free pages or slots: nothing was taken
    kUnknownRequest = -1,
    kAlreadyOpen = -2,
    kShrink = -3,         // a length smaller than the recorded one
    kNotReserved = -4,    // commit without the pages
    kBadPage = -5,        // a page given back that is not held
    kBadArgument = -6,
};

// Bookkeeping of the cache manager: per group a pool (and an optional window), per
// request a slot, a length and one page list per group (-1 where a windowed group
// gave the page back).
class CacheBook {
public:
    CacheBook(int n_groups, const int* windows, int page_size, const int* n_pages, int max_requests, bool track_fresh);

    int open(int64_t request);  // slot, kNoRoom as -100, or kAlreadyOpen
    bool is_open(int64_t request) const { return requests_.count(request) != 0; }
    int slot(int64_t request) const;
    int64_t length(int64_t request) const;
    int reserve(int64_t request, int64_t new_len);  // kOk, kNoRoom or an error
    int commit(int64_t request, int64_t new_len);
    int close(int64_t request);
    int pages_needed(int64_t request, int64_t new_len) const;
    // The request's page ids of `group` (with -1 holes) into out[0 .. capacity); returns the count.
    int table_row(int group, int64_t request, int32_t* out, int capacity) const;
    int held_pages(int group, int64_t request, int32_t* out, int capacity) const;
    int take_fresh(int group, int32_t* out, int capacity);
    int free_pages() const;  // of the fullest pool

    int n_groups() const { return static_cast<int>(pools_.size()); }
    int page_size() const { return page_size_; }
    int max_requests() const { return max_requests_; }
    int slots_used() const { return max_requests_ - static_cast<int>(free_slots_.size()); }
    const PagePool& pool(int group) const { return pools_[group]; }
    PagePool& pool(int group) { return pools_[group]; }
    std::vector<int64_t> open_requests() const;

private:
    struct Request {
        int slot = 0;
        int64_t length = 0;
        std::vector<std::vector<int>> pages;
    };
    int first_needed_page(int group, int64_t length) const;

    int page_size_;
    int max_requests_;
    bool track_fresh_;
    std::vector<int> windows_;
    std::vector<PagePool> pools_;
    std::vector<int> free_slots_;
    std::unordered_map<int64_t, Request> requests_;
    std::vector<int64_t> open_order_;
    std::vector<std::unordered_set<int>> fresh_;
};

// What the scheduler decides for one step.
struct PlannedEntry {
    int64_t request;
    int count;     // tokens of the request's pending list that run
    int samples;   // 1 when the step consumes all its pending tokens
};
struct Ended {
    int64_t request;
    int reason;    // Reason
};
enum Reason : int { kStop = 0, kLength = 1, kCancelled = 2, kOom = 3 };

// The scheduler's decisions (see pulsarlm_b200/engine/scheduler.py for the rules in
// words). It tracks counts only; token values stay with the caller.
class SchedulerCore {
public:
    SchedulerCore(CacheBook* cache, int prefill_tokens_per_step, int max_step_entries);
    void set_stop_ids(const int32_t* ids, int count);
    int add(int64_t request, int prompt_len, int64_t max_tokens, bool ignore_eos);
    int cancel(int64_t request);
    bool has_work() const { return !waiting_.empty() || !running_.empty(); }
    int preemptions() const { return preemptions_; }
    int preemptions_of(int64_t request) const;

    // Plans a step. Entries come single-token first. `preempted` lists requests sent
    // back to the queue (the caller rebuilds their pending tokens as prompt + output).
    void plan(std::vector<PlannedEntry>& entries, std::vector<Ended>& ended, std::vector<int64_t>& preempted);
    // A step in two halves, so that the next one can be planned while it runs: `advance` when it
    // leaves for the device (what it consumes is known), `settle` when its tokens are known
    // (tokens[i] is the token drawn for entries[i], ignored unless it samples).
    void advance(const PlannedEntry* entries, int count);
    void settle(const PlannedEntry* entries, const int32_t* tokens, int count, std::vector<Ended>& ended);
    // Both at once.
    void finish_step(const PlannedEntry* entries, const int32_t* tokens, int count, std::vector<Ended>& ended);

    std::vector<int64_t> running() const { return running_; }
    std::vector<int64_t> waiting() const { return {waiting_.begin(), waiting_.end()}; }

private:
    struct Request {
        int prompt_len = 0;
        int output_len = 0;  // tokens drawn and known
        int unsettled = 0;   // tokens being drawn by steps that have left and are not settled yet
        int pending = 0;
        int64_t max_tokens = -1;  // -1: no limit
        bool ignore_eos = false;
        bool cancelled = false;
        bool running = false;
        int preemptions = 0;
    };
    void finish(int64_t id, int reason, std::vector<Ended>& ended);
    void preempt(int64_t id, std::vector<int64_t>& preempted);
    bool reserve(int64_t id, int count, const std::unordered_set<int64_t>& planned, std::vector<int64_t>& preempted);
    bool is_running(int64_t id) const;

    CacheBook* cache_;
    int prefill_tokens_per_step_;
    int max_step_entries_;
    std::unordered_set<int32_t> stop_ids_;
    std::unordered_map<int64_t, Request> requests_;
    std::deque<int64_t> waiting_;
    std::vector<int64_t> running_;  // admission order
    int preemptions_ = 0;
};

}  // namespace plh
