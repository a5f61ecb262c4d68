// Implementation and C interface of the host core (see host_core.hpp).
#include "host_core.hpp"

#include <algorithm>

namespace plh {

// ------------------------------------------------------------------ PagePool

PagePool::PagePool(int n_pages) : held_(n_pages > 0 ? n_pages : 0, 0) {
    free_.reserve(held_.size());
    for (int page = static_cast<int>(held_.size()) - 1; page >= 0; --page) {
        free_.push_back(page);  // page 0 ends on top
    }
}

bool PagePool::take(int count, std::vector<int>& out) {
    if (count < 0 || count > free_count()) {
        return false;
    }
    for (int i = 0; i < count; ++i) {
        const int page = free_.back();
        free_.pop_back();
        held_[page] = 1;
        out.push_back(page);
    }
    high_water_ = std::max(high_water_, used_count());
    return true;
}

bool PagePool::give(const int* pages, int count) {
    for (int i = 0; i < count; ++i) {
        const int page = pages[i];
        if (!is_held(page)) {
            return false;
        }
        held_[page] = 0;
        free_.push_back(page);
    }
    return true;
}

// ------------------------------------------------------------------ CacheBook

CacheBook::CacheBook(int n_groups, const int* windows, int page_size, const int* n_pages, int max_requests,
                     bool track_fresh)
: page_size_(page_size), max_requests_(max_requests), track_fresh_(track_fresh) {
    for (int g = 0; g < n_groups; ++g) {
        windows_.push_back(windows != nullptr ? windows[g] : -1);
        pools_.emplace_back(n_pages[g]);  // (a group whose window lets pages go needs fewer than one that keeps all)
        fresh_.emplace_back();
    }
    for (int slot = max_requests - 1; slot >= 0; --slot) {
        free_slots_.push_back(slot);
    }
}

int CacheBook::open(int64_t request) {
    if (is_open(request)) {
        return kAlreadyOpen;
    }
    if (free_slots_.empty()) {
        return -100;
    }
    Request r;
    r.slot = free_slots_.back();
    free_slots_.pop_back();
    r.pages.resize(pools_.size());
    requests_.emplace(request, std::move(r));
    open_order_.push_back(request);
    return requests_[request].slot;
}

int CacheBook::slot(int64_t request) const {
    const auto it = requests_.find(request);
    return it == requests_.end() ? kUnknownRequest : it->second.slot;
}

int64_t CacheBook::length(int64_t request) const {
    const auto it = requests_.find(request);
    return it == requests_.end() ? kUnknownRequest : it->second.length;
}

int CacheBook::first_needed_page(int group, int64_t length) const {
    if (windows_[group] < 0) {
        return 0;
    }
    const int64_t first_key = std::max<int64_t>(0, length - windows_[group] + 1);
    return static_cast<int>(first_key / page_size_);
}

int CacheBook::pages_needed(int64_t request, int64_t new_len) const {
    const auto it = requests_.find(request);
    if (it == requests_.end()) {
        return kUnknownRequest;
    }
    const int64_t n_pages = (new_len + page_size_ - 1) / page_size_;
    int total = 0;
    for (size_t g = 0; g < pools_.size(); ++g) {
        total += static_cast<int>(std::max<int64_t>(0, n_pages - static_cast<int64_t>(it->second.pages[g].size())));
    }
    return total;
}

int CacheBook::reserve(int64_t request, int64_t new_len) {
    const auto it = requests_.find(request);
    if (it == requests_.end()) {
        return kUnknownRequest;
    }
    Request& r = it->second;
    if (new_len < r.length) {
        return kShrink;
    }
    const int64_t n_pages = (new_len + page_size_ - 1) / page_size_;
    std::vector<int> missing(pools_.size());
    for (size_t g = 0; g < pools_.size(); ++g) {
        missing[g] = static_cast<int>(std::max<int64_t>(0, n_pages - static_cast<int64_t>(r.pages[g].size())));
        if (missing[g] > pools_[g].free_count()) {
            return kNoRoom;
        }
    }
    for (size_t g = 0; g < pools_.size(); ++g) {
        const size_t before = r.pages[g].size();
        pools_[g].take(missing[g], r.pages[g]);
        if (track_fresh_) {
            fresh_[g].insert(r.pages[g].begin() + before, r.pages[g].end());
        }
    }
    return kOk;
}

int CacheBook::commit(int64_t request, int64_t new_len) {
    const auto it = requests_.find(request);
    if (it == requests_.end()) {
        return kUnknownRequest;
    }
    Request& r = it->second;
    const int64_t n_pages = (new_len + page_size_ - 1) / page_size_;
    if (new_len < r.length) {
        return kNotReserved;
    }
    for (const auto& pages : r.pages) {
        if (n_pages > static_cast<int64_t>(pages.size())) {
            return kNotReserved;
        }
    }
    r.length = new_len;
    for (size_t g = 0; g < pools_.size(); ++g) {
        std::vector<int>& pages = r.pages[g];
        const int first = std::min<int>(first_needed_page(static_cast<int>(g), new_len), static_cast<int>(pages.size()));
        for (int i = 0; i < first; ++i) {
            if (pages[i] >= 0) {
                if (!pools_[g].give(&pages[i], 1)) {
                    return kBadPage;
                }
                pages[i] = -1;
            }
        }
    }
    return kOk;
}

int CacheBook::close(int64_t request) {
    const auto it = requests_.find(request);
    if (it == requests_.end()) {
        return kUnknownRequest;
    }
    int code = kOk;
    for (size_t g = 0; g < pools_.size(); ++g) {
        for (int page : it->second.pages[g]) {
            if (page >= 0 && !pools_[g].give(&page, 1)) {
                code = kBadPage;
            }
        }
    }
    free_slots_.push_back(it->second.slot);
    requests_.erase(it);
    open_order_.erase(std::find(open_order_.begin(), open_order_.end(), request));
    return code;
}

int CacheBook::table_row(int group, int64_t request, int32_t* out, int capacity) const {
    const auto it = requests_.find(request);
    if (it == requests_.end() || group < 0 || group >= n_groups()) {
        return kUnknownRequest;
    }
    const std::vector<int>& pages = it->second.pages[group];
    const int n = static_cast<int>(pages.size());
    for (int i = 0; i < n && i < capacity; ++i) {
        out[i] = pages[i];
    }
    return n;
}

int CacheBook::held_pages(int group, int64_t request, int32_t* out, int capacity) const {
    const auto it = requests_.find(request);
    if (it == requests_.end() || group < 0 || group >= n_groups()) {
        return kUnknownRequest;
    }
    int n = 0;
    for (int page : it->second.pages[group]) {
        if (page >= 0) {
            if (n < capacity) {
                out[n] = page;
            }
            ++n;
        }
    }
    return n;
}

int CacheBook::take_fresh(int group, int32_t* out, int capacity) {
    int n = 0;
    for (int page : fresh_[group]) {
        if (n < capacity) {
            out[n] = page;
        }
        ++n;
    }
    if (n <= capacity) {
        fresh_[group].clear();
    }
    return n;
}

int CacheBook::free_pages() const {
    int least = pools_.empty() ? 0 : pools_[0].free_count();
    for (const PagePool& pool : pools_) {
        least = std::min(least, pool.free_count());
    }
    return least;
}

std::vector<int64_t> CacheBook::open_requests() const { return open_order_; }

// ------------------------------------------------------------------ SchedulerCore

SchedulerCore::SchedulerCore(CacheBook* cache, int prefill_tokens_per_step, int max_step_entries)
: cache_(cache), prefill_tokens_per_step_(prefill_tokens_per_step), max_step_entries_(max_step_entries) {}

void SchedulerCore::set_stop_ids(const int32_t* ids, int count) {
    stop_ids_.clear();
    stop_ids_.insert(ids, ids + count);
}

int SchedulerCore::add(int64_t request, int prompt_len, int64_t max_tokens, bool ignore_eos) {
    if (prompt_len <= 0 || requests_.count(request)) {
        return kBadArgument;
    }
    Request r;
    r.prompt_len = prompt_len;
    r.pending = prompt_len;
    r.max_tokens = max_tokens;
    r.ignore_eos = ignore_eos;
    requests_.emplace(request, r);
    waiting_.push_back(request);
    return kOk;
}

int SchedulerCore::cancel(int64_t request) {
    const auto it = requests_.find(request);
    if (it == requests_.end()) {
        return kUnknownRequest;
    }
    it->second.cancelled = true;
    return kOk;
}

int SchedulerCore::preemptions_of(int64_t request) const {
    const auto it = requests_.find(request);
    return it == requests_.end() ? 0 : it->second.preemptions;
}

bool SchedulerCore::is_running(int64_t id) const {
    return std::find(running_.begin(), running_.end(), id) != running_.end();
}

void SchedulerCore::finish(int64_t id, int reason, std::vector<Ended>& ended) {
    if (cache_->is_open(id)) {
        cache_->close(id);
    }
    const auto at = std::find(running_.begin(), running_.end(), id);
    if (at != running_.end()) {
        running_.erase(at);
    }
    requests_.erase(id);
    ended.push_back({id, reason});
}

void SchedulerCore::preempt(int64_t id, std::vector<int64_t>& preempted) {
    Request& r = requests_[id];
    cache_->close(id);
    running_.erase(std::find(running_.begin(), running_.end(), id));
    r.pending = r.prompt_len + r.output_len;  // everything it computed is recomputed later
    r.unsettled = 0;                          // (a token still being drawn is dropped and drawn again)
    r.running = false;
    ++r.preemptions;
    ++preemptions_;
    waiting_.push_front(id);
    preempted.push_back(id);
}

// Pages for `count` more tokens of a running request, preempting the newest other
// running request (never one already planned) while that helps.
bool SchedulerCore::reserve(int64_t id, int count, const std::unordered_set<int64_t>& planned,
                            std::vector<int64_t>& preempted) {
    const int64_t new_len = cache_->length(id) + count;
    while (cache_->reserve(id, new_len) != kOk) {
        int64_t victim = 0;
        bool found = false;
        for (auto it = running_.rbegin(); it != running_.rend(); ++it) {
            if (*it != id && !planned.count(*it)) {
                victim = *it;
                found = true;
                break;
            }
        }
        if (!found) {
            return false;
        }
        preempt(victim, preempted);
    }
    return true;
}

void SchedulerCore::plan(std::vector<PlannedEntry>& entries, std::vector<Ended>& ended,
                         std::vector<int64_t>& preempted) {
    // cancelled requests leave first
    for (const int64_t id : std::vector<int64_t>(running_)) {
        if (requests_[id].cancelled) {
            finish(id, kCancelled, ended);
        }
    }
    for (const int64_t id : std::vector<int64_t>(waiting_.begin(), waiting_.end())) {
        if (requests_[id].cancelled) {
            waiting_.erase(std::find(waiting_.begin(), waiting_.end(), id));
            finish(id, kCancelled, ended);
        }
    }
    std::unordered_set<int64_t> planned;
    std::vector<PlannedEntry> prompt_entries;

    // 1. decoding requests, oldest first; a preempted one simply leaves `running_`.
    for (const int64_t id : std::vector<int64_t>(running_)) {
        if (!is_running(id) || requests_[id].pending != 1) {
            continue;
        }
        if (static_cast<int>(entries.size()) >= max_step_entries_) {
            break;
        }
        if (reserve(id, 1, planned, preempted)) {
            entries.push_back({id, 1, 1});
            planned.insert(id);
        } else if (planned.empty() && running_.size() == 1) {
            finish(id, kOom, ended);
        }
    }
    // 2. prompt portions of running requests, then of newly admitted ones.
    int budget = prefill_tokens_per_step_;
    auto room = [&] { return static_cast<int>(entries.size() + prompt_entries.size()) < max_step_entries_; };
    for (const int64_t id : std::vector<int64_t>(running_)) {
        if (budget == 0 || !room()) {
            break;
        }
        if (!is_running(id) || requests_[id].pending <= 1 || planned.count(id)) {
            continue;
        }
        const int count = std::min(requests_[id].pending, budget);
        if (reserve(id, count, planned, preempted)) {
            prompt_entries.push_back({id, count, count == requests_[id].pending ? 1 : 0});
            planned.insert(id);
            budget -= count;
        } else if (planned.empty() && running_.size() == 1) {
            finish(id, kOom, ended);
        }
    }
    while (!waiting_.empty() && budget > 0 && room()) {
        const int64_t id = waiting_.front();
        Request& r = requests_[id];
        const int count = std::min(r.pending, budget);
        if (cache_->open(id) < 0) {
            break;
        }
        if (cache_->reserve(id, count) != kOk) {
            cache_->close(id);
            if (running_.empty()) {
                // Alone and still too large for the pool: it can never run.
                waiting_.pop_front();
                finish(id, kOom, ended);
                continue;
            }
            break;
        }
        waiting_.pop_front();
        r.running = true;
        running_.push_back(id);
        prompt_entries.push_back({id, count, count == r.pending ? 1 : 0});
        planned.insert(id);
        budget -= count;
    }
    // single-token entries first (stable), as the kernels' launchers like it
    std::vector<PlannedEntry> singles, others;
    for (const PlannedEntry& e : prompt_entries) {
        (e.count == 1 ? singles : others).push_back(e);
    }
    entries.insert(entries.end(), singles.begin(), singles.end());
    entries.insert(entries.end(), others.begin(), others.end());
}

// A step leaves for the device. Its prompt tokens are consumed; a request that samples in it
// is taken to go on with the token being drawn (one pending token, not yet known to the host),
// unless that token is certain to be its last: then nothing is planned for it until `settle`.
void SchedulerCore::advance(const PlannedEntry* entries, int count) {
    for (int i = 0; i < count; ++i) {
        const auto it = requests_.find(entries[i].request);
        if (it == requests_.end() || !it->second.running) {
            continue;
        }
        Request& r = it->second;
        r.pending -= entries[i].count;
        if (!entries[i].samples) {
            continue;
        }
        if (r.max_tokens == 0) {
            r.pending = 0;
            continue;
        }
        ++r.unsettled;
        r.pending = (r.max_tokens >= 0 && r.output_len + r.unsettled >= r.max_tokens) ? 0 : 1;
    }
}

// The tokens of a step that `advance` saw are known. The caller leaves out entries whose
// request was preempted or ended since the step left.
void SchedulerCore::settle(const PlannedEntry* entries, const int32_t* tokens, int count, std::vector<Ended>& ended) {
    for (int i = 0; i < count; ++i) {
        const int64_t id = entries[i].request;
        const auto it = requests_.find(id);
        if (it == requests_.end() || !it->second.running || !entries[i].samples) {
            continue;
        }
        Request& r = it->second;
        if (r.max_tokens == 0) {
            finish(id, kLength, ended);
            continue;
        }
        if (r.unsettled > 0) {
            --r.unsettled;
        }
        ++r.output_len;
        if (stop_ids_.count(tokens[i]) && !r.ignore_eos) {
            finish(id, kStop, ended);  // (what a later step in flight computes for it is dropped)
        } else if (r.max_tokens >= 0 && r.output_len >= r.max_tokens) {
            finish(id, kLength, ended);
        }
    }
}

void SchedulerCore::finish_step(const PlannedEntry* entries, const int32_t* tokens, int count,
                                std::vector<Ended>& ended) {
    advance(entries, count);
    settle(entries, tokens, count, ended);
}

}  // namespace plh

// ------------------------------------------------------------------ C interface

#define PLH_API extern "C" __attribute__((visibility("default")))

using plh::CacheBook;
using plh::PagePool;
using plh::SchedulerCore;

PLH_API int plh_abi_version() { return 5; }

PLH_API void* plh_pool_create(int n_pages) { return new PagePool(n_pages); }
PLH_API void plh_pool_destroy(void* pool) { delete static_cast<PagePool*>(pool); }
PLH_API int plh_pool_take(void* pool, int count, int32_t* out) {
    std::vector<int> taken;
    if (!static_cast<PagePool*>(pool)->take(count, taken)) {
        return -1;
    }
    std::copy(taken.begin(), taken.end(), out);
    return count;
}
PLH_API int plh_pool_give(void* pool, const int32_t* pages, int count) {
    return static_cast<PagePool*>(pool)->give(pages, count) ? 0 : plh::kBadPage;
}
// what: 0 pages, 1 free, 2 used, 3 high water
PLH_API int plh_pool_stat(void* pool, int what) {
    const PagePool* p = static_cast<PagePool*>(pool);
    return what == 0 ? p->n_pages() : what == 1 ? p->free_count() : what == 2 ? p->used_count() : p->high_water();
}
PLH_API int plh_pool_is_held(void* pool, int page) { return static_cast<PagePool*>(pool)->is_held(page) ? 1 : 0; }

PLH_API void* plh_cache_create(int n_groups, const int32_t* windows, int page_size, const int32_t* n_pages,
                               int max_requests, int track_fresh) {
    return new CacheBook(n_groups, windows, page_size, n_pages, max_requests, track_fresh != 0);
}
PLH_API void plh_cache_destroy(void* cache) { delete static_cast<CacheBook*>(cache); }
PLH_API int plh_cache_open(void* cache, int64_t request) { return static_cast<CacheBook*>(cache)->open(request); }
PLH_API int plh_cache_is_open(void* cache, int64_t request) {
    return static_cast<CacheBook*>(cache)->is_open(request) ? 1 : 0;
}
PLH_API int plh_cache_slot(void* cache, int64_t request) { return static_cast<CacheBook*>(cache)->slot(request); }
PLH_API int64_t plh_cache_length(void* cache, int64_t request) {
    return static_cast<CacheBook*>(cache)->length(request);
}
PLH_API int plh_cache_reserve(void* cache, int64_t request, int64_t new_len) {
    return static_cast<CacheBook*>(cache)->reserve(request, new_len);
}
PLH_API int plh_cache_commit(void* cache, int64_t request, int64_t new_len) {
    return static_cast<CacheBook*>(cache)->commit(request, new_len);
}
PLH_API int plh_cache_close(void* cache, int64_t request) { return static_cast<CacheBook*>(cache)->close(request); }
PLH_API int plh_cache_pages_needed(void* cache, int64_t request, int64_t new_len) {
    return static_cast<CacheBook*>(cache)->pages_needed(request, new_len);
}
PLH_API int plh_cache_table_row(void* cache, int group, int64_t request, int32_t* out, int capacity) {
    return static_cast<CacheBook*>(cache)->table_row(group, request, out, capacity);
}
PLH_API int plh_cache_held_pages(void* cache, int group, int64_t request, int32_t* out, int capacity) {
    return static_cast<CacheBook*>(cache)->held_pages(group, request, out, capacity);
}
PLH_API int plh_cache_take_fresh(void* cache, int group, int32_t* out, int capacity) {
    return static_cast<CacheBook*>(cache)->take_fresh(group, out, capacity);
}
PLH_API int plh_cache_free_pages(void* cache) { return static_cast<CacheBook*>(cache)->free_pages(); }
PLH_API int plh_cache_slots_used(void* cache) { return static_cast<CacheBook*>(cache)->slots_used(); }
// what as plh_pool_stat
PLH_API int plh_cache_pool_stat(void* cache, int group, int what) {
    const PagePool& p = static_cast<CacheBook*>(cache)->pool(group);
    return what == 0 ? p.n_pages() : what == 1 ? p.free_count() : what == 2 ? p.used_count() : p.high_water();
}
PLH_API int plh_cache_pool_is_held(void* cache, int group, int page) {
    return static_cast<CacheBook*>(cache)->pool(group).is_held(page) ? 1 : 0;
}
PLH_API int plh_cache_open_requests(void* cache, int64_t* out, int capacity) {
    const std::vector<int64_t> ids = static_cast<CacheBook*>(cache)->open_requests();
    for (size_t i = 0; i < ids.size() && static_cast<int>(i) < capacity; ++i) {
        out[i] = ids[i];
    }
    return static_cast<int>(ids.size());
}
// Fills rows of a [count, width] int32 table (-1 where a request holds no page) and
// each request's slot; returns the longest row, or an error code.
PLH_API int plh_cache_fill_tables(void* cache, int group, const int64_t* requests, int count, int32_t* table,
                                  int width, int32_t* slots) {
    const CacheBook* book = static_cast<CacheBook*>(cache);
    int longest = 0;
    for (int i = 0; i < count; ++i) {
        int32_t* row = table + static_cast<int64_t>(i) * width;
        std::fill(row, row + width, -1);
        const int n = book->table_row(group, requests[i], row, width);
        if (n < 0) {
            return n;
        }
        longest = std::max(longest, n);
        if (slots != nullptr) {
            slots[i] = book->slot(requests[i]);
        }
    }
    return longest;
}

// A step's entries in one call. For entry i: lens[i] = tokens request i holds, slots[i] =
// its slot, then pages are reserved for lens[i] + n_new[i] tokens. Returns the number of
// entries done: `count`, or fewer, with *code the code that stopped entry [return value]
// (kNoRoom: too few pages; reservations made for the entries before it stay).
PLH_API int plh_cache_reserve_many(void* cache, const int64_t* requests, const int32_t* n_new, int count,
                                   int64_t* lens, int32_t* slots, int32_t* code) {
    auto* book = static_cast<CacheBook*>(cache);
    *code = plh::kOk;
    for (int i = 0; i < count; ++i) {
        if (!book->is_open(requests[i])) {
            *code = plh::kUnknownRequest;
            return i;
        }
        lens[i] = book->length(requests[i]);
        slots[i] = book->slot(requests[i]);
        const int result = book->reserve(requests[i], lens[i] + n_new[i]);
        if (result != plh::kOk) {
            *code = result;
            return i;
        }
    }
    return count;
}

// commit(request i, new_lens[i]) for every entry; the first error code, or kOk.
PLH_API int plh_cache_commit_many(void* cache, const int64_t* requests, const int64_t* new_lens, int count) {
    auto* book = static_cast<CacheBook*>(cache);
    for (int i = 0; i < count; ++i) {
        const int result = book->commit(requests[i], new_lens[i]);
        if (result != plh::kOk) {
            return result;
        }
    }
    return plh::kOk;
}

PLH_API void* plh_sched_create(void* cache, int prefill_tokens_per_step, int max_step_entries) {
    return new SchedulerCore(static_cast<CacheBook*>(cache), prefill_tokens_per_step, max_step_entries);
}
PLH_API void plh_sched_destroy(void* sched) { delete static_cast<SchedulerCore*>(sched); }
PLH_API void plh_sched_set_stop_ids(void* sched, const int32_t* ids, int count) {
    static_cast<SchedulerCore*>(sched)->set_stop_ids(ids, count);
}
PLH_API int plh_sched_add(void* sched, int64_t request, int prompt_len, int64_t max_tokens, int ignore_eos) {
    return static_cast<SchedulerCore*>(sched)->add(request, prompt_len, max_tokens, ignore_eos != 0);
}
PLH_API int plh_sched_cancel(void* sched, int64_t request) { return static_cast<SchedulerCore*>(sched)->cancel(request); }
PLH_API int plh_sched_has_work(void* sched) { return static_cast<SchedulerCore*>(sched)->has_work() ? 1 : 0; }
PLH_API int plh_sched_preemptions(void* sched) { return static_cast<SchedulerCore*>(sched)->preemptions(); }
// Plans a step. entries: [capacity][3] = request, count, samples; ended: [capacity][2]
// = request, reason; preempted: [capacity]. counts: out[3] = entries, ended, preempted.
PLH_API int plh_sched_plan(void* sched, int64_t* entries, int64_t* ended, int64_t* preempted, int capacity,
                           int32_t* counts) {
    std::vector<plh::PlannedEntry> e;
    std::vector<plh::Ended> x;
    std::vector<int64_t> p;
    static_cast<SchedulerCore*>(sched)->plan(e, x, p);
    if (static_cast<int>(e.size()) > capacity || static_cast<int>(x.size()) > capacity ||
        static_cast<int>(p.size()) > capacity) {
        return plh::kBadArgument;
    }
    for (size_t i = 0; i < e.size(); ++i) {
        entries[3 * i] = e[i].request;
        entries[3 * i + 1] = e[i].count;
        entries[3 * i + 2] = e[i].samples;
    }
    for (size_t i = 0; i < x.size(); ++i) {
        ended[2 * i] = x[i].request;
        ended[2 * i + 1] = x[i].reason;
    }
    std::copy(p.begin(), p.end(), preempted);
    counts[0] = static_cast<int32_t>(e.size());
    counts[1] = static_cast<int32_t>(x.size());
    counts[2] = static_cast<int32_t>(p.size());
    return 0;
}
// entries as plh_sched_plan wrote them; tokens[count]; ended: [capacity][2]. Returns how many ended.
PLH_API int plh_sched_finish_step(void* sched, const int64_t* entries, const int32_t* tokens, int count,
                                  int64_t* ended, int capacity) {
    std::vector<plh::PlannedEntry> e(count);
    for (int i = 0; i < count; ++i) {
        e[i] = {entries[3 * i], static_cast<int>(entries[3 * i + 1]), static_cast<int>(entries[3 * i + 2])};
    }
    std::vector<plh::Ended> x;
    static_cast<SchedulerCore*>(sched)->finish_step(e.data(), tokens, count, x);
    for (size_t i = 0; i < x.size() && static_cast<int>(i) < capacity; ++i) {
        ended[2 * i] = x[i].request;
        ended[2 * i + 1] = x[i].reason;
    }
    return static_cast<int>(x.size());
}

PLH_API void plh_sched_advance(void* sched, const int64_t* entries, int count) {
    std::vector<plh::PlannedEntry> e(count);
    for (int i = 0; i < count; ++i) {
        e[i] = {entries[3 * i], static_cast<int>(entries[3 * i + 1]), static_cast<int>(entries[3 * i + 2])};
    }
    static_cast<SchedulerCore*>(sched)->advance(e.data(), count);
}
PLH_API int plh_sched_settle(void* sched, const int64_t* entries, const int32_t* tokens, int count, int64_t* ended,
                             int capacity) {
    std::vector<plh::PlannedEntry> e(count);
    for (int i = 0; i < count; ++i) {
        e[i] = {entries[3 * i], static_cast<int>(entries[3 * i + 1]), static_cast<int>(entries[3 * i + 2])};
    }
    std::vector<plh::Ended> x;
    static_cast<SchedulerCore*>(sched)->settle(e.data(), tokens, count, x);
    for (size_t i = 0; i < x.size() && static_cast<int>(i) < capacity; ++i) {
        ended[2 * i] = x[i].request;
        ended[2 * i + 1] = x[i].reason;
    }
    return static_cast<int>(x.size());
}

// ---------------------------------------------------------------------------
// Random weights on the host (the device's twin is pl_fill_random; same bits).
#include "../csrc/random_values.h"

// out (fp32 when dtype is 0, bfloat16 bits when 1; n elements) = offset + scale * noise,
// the noise a function of (seed, tensor_hash, element index) alone.
PLH_API int plh_fill_random(void* out, int64_t n, int dtype, uint64_t seed, uint64_t tensor_hash, float scale,
                            float offset) {
    if (n < 0 || (dtype != 0 && dtype != 1) || (out == nullptr && n > 0)) {
        return plh::kBadArgument;
    }
    const uint64_t key = pl_random_key(seed, tensor_hash);
    if (dtype == 0) {
        float* values = static_cast<float*>(out);
        for (int64_t i = 0; i < n; ++i) {
            values[i] = pl_random_value(key, static_cast<uint64_t>(i), scale, offset);
        }
    } else {
        uint16_t* values = static_cast<uint16_t*>(out);
        for (int64_t i = 0; i < n; ++i) {
            values[i] = pl_random_bf16_bits(pl_random_value(key, static_cast<uint64_t>(i), scale, offset));
        }
    }
    return 0;
}

// ---------------------------------------------------------------------------
// The work list of a step's single tokens for the decode attention kernel.
//
// lengths[n]: keys each token's request holds after the step; window: 0 or how many of
// the last keys a query reads. The tokens' 16-key tiles are cut into about `target` items
// of equal size (none much shorter than min_tiles), a request's share rounded to whole
// items that differ by one tile at most; requests of about one length (longest within
// even_percent of the mean) are left whole. Rows {token, first tile, tiles, split | splits
// << 12}, longest first, go to items[capacity][4]; unused rows are zero and the last of
// them holds the number of rows in use in its first field. slots[n]: first scratch slot of
// each token's splits. Returns the number of rows in use, or a negative code when
// `capacity` is too small (at most target + n are needed).
PLH_API int plh_decode_work_items(const int32_t* lengths, int n, int window, int target, int min_tiles,
                                  int even_percent, int32_t* items, int capacity, int32_t* slots) {
    if (n < 0 || target < 1 || min_tiles < 1 || capacity < 1 || lengths == nullptr || items == nullptr ||
        slots == nullptr) {
        return plh::kBadArgument;
    }
    struct Row {
        int32_t token, first, tiles, code;
    };
    std::vector<Row> rows;
    rows.reserve(static_cast<size_t>(n) + target);
    int64_t total = 0;
    int32_t longest = 0;
    std::vector<int32_t> first(n), tiles(n);
    for (int t = 0; t < n; ++t) {
        const int32_t context = lengths[t];
        first[t] = (window > 0 && context > window ? context - window : 0) / 16;
        tiles[t] = std::max<int32_t>(0, (context + 15) / 16 - first[t]);
        total += tiles[t];
        longest = std::max(longest, tiles[t]);
    }
    const int64_t chunk = std::max<int64_t>(min_tiles, (total + target - 1) / target);
    const bool even = static_cast<int64_t>(longest) * n * 100 <= static_cast<int64_t>(even_percent) * total;
    int32_t slot = 0;
    for (int t = 0; t < n; ++t) {
        int64_t k = even ? 1 : (2 * static_cast<int64_t>(tiles[t]) + chunk) / (2 * chunk);  // tiles / chunk, rounded
        k = std::min<int64_t>(4095, std::max<int64_t>(1, k));
        slots[t] = slot;
        if (k > 1) {
            slot += static_cast<int32_t>(k);
        }
        int32_t at = first[t];
        for (int32_t s = 0; s < k; ++s) {
            const int32_t share = tiles[t] / static_cast<int32_t>(k) + (s < tiles[t] % static_cast<int32_t>(k) ? 1 : 0);
            rows.push_back({t, at, share, s | (static_cast<int32_t>(k) << 12)});
            at += share;
        }
    }
    std::stable_sort(rows.begin(), rows.end(), [](const Row& a, const Row& b) { return a.tiles > b.tiles; });
    if (static_cast<int>(rows.size()) > capacity) {
        return plh::kBadArgument;
    }
    std::fill(items, items + static_cast<size_t>(capacity) * 4, 0);
    for (size_t i = 0; i < rows.size(); ++i) {
        items[4 * i] = rows[i].token;
        items[4 * i + 1] = rows[i].first;
        items[4 * i + 2] = rows[i].tiles;
        items[4 * i + 3] = rows[i].code;
    }
    if (static_cast<int>(rows.size()) < capacity) {
        items[4 * (capacity - 1)] = static_cast<int32_t>(rows.size());
    }
    return static_cast<int>(rows.size());
}
