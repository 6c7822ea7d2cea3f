// The host-side runtime: the paged cache's books (page pools, per-request block tables, the
// mirror of the tables that the step function uploads, request slots) and the scheduler that
// decides each step's batch.  Plain C++17, no CUDA; exported as C functions over opaque handles
// (the Python classes of nanoinfer_b200.cache and nanoinfer_b200.engine.scheduler are thin
// wrappers).  Every function returns 0 / a count, or a negative code with a message kept in the
// object (ni_cache_last_error); a refused call changes nothing.
//
// A *group* is a set of layer runs with the same need (kv heads, head size, window).  Each group
// has its own page pool and, per request, its own block table; pages are taken on demand
// (append), given back when a request ends (free) and, in a windowed group, as soon as the window
// has passed them (release_passed).
//
// Reference counterparts: BlockManager (src/engine/block_manager.cpp:17-182: LIFO stack whose
// first pops are 0, 1, 2, ..., allocated bitmap, double-free and range errors), BlockTable
// (src/engine/block_table.cpp:22-221: rebuilt and flattened every step) and KVCacheManager
// (src/engine/kv_cache_manager.cpp:120-220: one group, whole prompt reserved at admission,
// everything given back at the end).
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <deque>
#include <string>
#include <unordered_map>
#include <vector>

#define NI_HOST_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

constexpr int kOk = 0;
constexpr int kErrArgument = -1;     // bad argument or unknown request
constexpr int kErrOutOfPages = -2;   // the pool has too few free pages; nothing was taken
constexpr int kErrPage = -3;         // page out of range, not held, or freed twice
constexpr int kErrLimit = -4;        // the request would exceed max_tokens_per_request
constexpr int kErrNoSlot = -5;       // no free request slot
constexpr int kErrInconsistent = -6; // check_consistency found a fault

struct PagePool {
    int num_pages;
    std::vector<int32_t> free_stack;   // top = next page handed out
    std::vector<uint8_t> taken;
    std::string error;

    explicit PagePool(int n) : num_pages(n), taken((size_t)n, 0) {
        free_stack.reserve((size_t)n);
        for (int p = n - 1; p >= 0; --p) free_stack.push_back(p);   // first pops are 0, 1, 2, ...
    }
    int num_free() const { return (int)free_stack.size(); }
    bool is_taken(int p) const { return p >= 0 && p < num_pages && taken[(size_t)p]; }

    int take(int n, int32_t* out) {
        if (n < 0) { error = "cannot take a negative number of pages"; return kErrArgument; }
        if (n > num_free()) {
            error = "asked for " + std::to_string(n) + " pages, " + std::to_string(num_free()) + " of " +
                    std::to_string(num_pages) + " are free";
            return kErrOutOfPages;
        }
        for (int i = 0; i < n; ++i) {
            const int32_t p = free_stack.back();
            free_stack.pop_back();
            taken[(size_t)p] = 1;
            out[i] = p;
        }
        return kOk;
    }
    // All or nothing: a page out of range, not held, or named twice refuses the whole call.
    int give_back(const int32_t* pages, int n) {
        for (int i = 0; i < n; ++i) {
            const int32_t p = pages[i];
            if (p < 0 || p >= num_pages) {
                error = "page " + std::to_string(p) + " is outside the pool of " + std::to_string(num_pages);
                return kErrPage;
            }
            if (!taken[(size_t)p]) { error = "page " + std::to_string(p) + " is not held (freed twice?)"; return kErrPage; }
            for (int j = 0; j < i; ++j)
                if (pages[j] == p) { error = "page " + std::to_string(p) + " is not held (freed twice?)"; return kErrPage; }
        }
        for (int i = 0; i < n; ++i) {
            taken[(size_t)pages[i]] = 0;
            free_stack.push_back(pages[i]);
        }
        return kOk;
    }
};

struct Held {
    int slot = 0;
    int length = 0;                                // tokens whose keys/values are (being) cached
    std::vector<std::vector<int32_t>> tables;      // per group; -1 = released
    std::vector<int> first_live;                   // per group: first page not yet released
};

struct CacheManager {
    int page_size, max_requests, max_tokens, table_width;
    std::vector<int> windows;                      // per group, -1 = all keys
    std::vector<PagePool> pools;
    std::vector<std::vector<int32_t>> mirror;      // per group [max_requests * table_width], -1 = no page
    std::vector<int> free_slots;
    std::unordered_map<long long, Held> held;
    long long table_version = 0;                   // bumped whenever a row of the mirror changes
    bool windowed = false;
    std::string error;

    CacheManager(int n_groups, const int* pages, const int* win, int page, int max_req, int max_tok)
        : page_size(page), max_requests(max_req), max_tokens(max_tok), table_width((max_tok + page - 1) / page) {
        for (int g = 0; g < n_groups; ++g) {
            windows.push_back(win[g]);
            windowed = windowed || win[g] >= 0;
            pools.emplace_back(pages[g]);
            mirror.emplace_back((size_t)max_req * table_width, -1);
        }
        for (int s = max_req - 1; s >= 0; --s) free_slots.push_back(s);
    }
    int n_groups() const { return (int)pools.size(); }

    Held* get(long long req) {
        auto it = held.find(req);
        if (it == held.end()) { error = "request is not admitted"; return nullptr; }
        return &it->second;
    }
    int32_t* row(int g, int slot) { return mirror[(size_t)g].data() + (size_t)slot * table_width; }

    int admit(long long req) {
        if (held.count(req)) { error = "request is already admitted"; return kErrArgument; }
        if (free_slots.empty()) { error = "no free request slot"; return kErrNoSlot; }
        const int slot = free_slots.back();
        free_slots.pop_back();
        Held h;
        h.slot = slot;
        h.tables.resize((size_t)n_groups());
        h.first_live.assign((size_t)n_groups(), 0);
        held.emplace(req, std::move(h));
        for (int g = 0; g < n_groups(); ++g)
            for (int i = 0; i < table_width; ++i) row(g, slot)[i] = -1;
        ++table_version;
        return slot;
    }
    // Pages each group must still take so that n_new more tokens fit.
    void pages_needed(const Held& h, int n_new, int* out) const {
        const int total = (h.length + n_new + page_size - 1) / page_size;
        for (int g = 0; g < n_groups(); ++g) out[g] = total - (int)h.tables[(size_t)g].size();
    }
    int append(long long req, int n_new) {
        Held* h = get(req);
        if (!h) return kErrArgument;
        if (n_new < 0) { error = "n_new must not be negative"; return kErrArgument; }
        if (h->length + n_new > max_tokens) {
            error = "request would hold " + std::to_string(h->length + n_new) + " tokens, more than max_tokens_per_request " +
                    std::to_string(max_tokens);
            return kErrLimit;
        }
        std::vector<int> need((size_t)n_groups());
        pages_needed(*h, n_new, need.data());
        for (int g = 0; g < n_groups(); ++g)
            if (need[(size_t)g] > pools[(size_t)g].num_free()) {
                error = "group " + std::to_string(g) + ": request needs " + std::to_string(need[(size_t)g]) +
                        " more pages, " + std::to_string(pools[(size_t)g].num_free()) + " are free";
                return kErrOutOfPages;
            }
        for (int g = 0; g < n_groups(); ++g) {
            const int n = need[(size_t)g];
            if (n <= 0) continue;
            auto& table = h->tables[(size_t)g];
            const size_t start = table.size();
            table.resize(start + (size_t)n);
            pools[(size_t)g].take(n, table.data() + start);
            for (int i = 0; i < n; ++i) row(g, h->slot)[start + (size_t)i] = table[start + (size_t)i];
            ++table_version;
        }
        h->length += n_new;
        return kOk;
    }
    int first_needed_page(int g, int length) const {   // first page a query at position >= length can still see
        const int w = windows[(size_t)g];
        if (w < 0) return 0;
        const int lo = length - w + 1;
        return (lo > 0 ? lo : 0) / page_size;
    }
    int release_passed(long long req) {
        if (!windowed) return held.count(req) ? 0 : (error = "request is not admitted", kErrArgument);
        Held* h = get(req);
        if (!h) return kErrArgument;
        int released = 0;
        for (int g = 0; g < n_groups(); ++g) {
            if (windows[(size_t)g] < 0) continue;
            auto& table = h->tables[(size_t)g];
            int first = first_needed_page(g, h->length);
            if (first > (int)table.size()) first = (int)table.size();
            const int live = h->first_live[(size_t)g];
            if (first > live) {
                const int rc = pools[(size_t)g].give_back(table.data() + live, first - live);
                if (rc != kOk) { error = pools[(size_t)g].error; return rc; }
                for (int i = live; i < first; ++i) { table[(size_t)i] = -1; row(g, h->slot)[i] = -1; }
                ++table_version;
                released += first - live;
                h->first_live[(size_t)g] = first;
            }
        }
        return released;
    }
    int free_request(long long req) {
        Held* h = get(req);
        if (!h) return kErrArgument;
        for (int g = 0; g < n_groups(); ++g) {
            std::vector<int32_t> pages;
            for (int32_t p : h->tables[(size_t)g])
                if (p >= 0) pages.push_back(p);
            const int rc = pools[(size_t)g].give_back(pages.data(), (int)pages.size());
            if (rc != kOk) { error = pools[(size_t)g].error; return rc; }
            for (int i = 0; i < table_width; ++i) row(g, h->slot)[i] = -1;
        }
        ++table_version;
        free_slots.push_back(h->slot);
        held.erase(req);
        return kOk;
    }
    // Every taken page is held by exactly one request, nothing else is taken, slots add up.
    int check() {
        for (int g = 0; g < n_groups(); ++g) {
            std::vector<uint8_t> seen((size_t)pools[(size_t)g].num_pages, 0);
            int n_held = 0;
            for (auto& kv : held)
                for (int32_t p : kv.second.tables[(size_t)g]) {
                    if (p < 0) continue;
                    if (p >= pools[(size_t)g].num_pages || seen[(size_t)p]) {
                        error = "group " + std::to_string(g) + ": a page is held twice";
                        return kErrInconsistent;
                    }
                    if (!pools[(size_t)g].is_taken(p)) {
                        error = "group " + std::to_string(g) + ": a held page is not marked taken";
                        return kErrInconsistent;
                    }
                    seen[(size_t)p] = 1;
                    ++n_held;
                }
            const int taken = pools[(size_t)g].num_pages - pools[(size_t)g].num_free();
            if (n_held != taken) {
                error = "group " + std::to_string(g) + ": " + std::to_string(taken) + " pages taken, " +
                        std::to_string(n_held) + " held";
                return kErrInconsistent;
            }
        }
        std::vector<uint8_t> slot_seen((size_t)max_requests, 0);
        for (auto& kv : held) {
            const int s = kv.second.slot;
            if (s < 0 || s >= max_requests || slot_seen[(size_t)s]) { error = "request slots are inconsistent"; return kErrInconsistent; }
            slot_seen[(size_t)s] = 1;
        }
        if ((int)held.size() + (int)free_slots.size() != max_requests) { error = "request slots are inconsistent"; return kErrInconsistent; }
        return kOk;
    }
};

}  // namespace

// ---- page pool -----------------------------------------------------------------------------------
NI_HOST_EXPORT void* ni_pool_create(int num_pages) { return num_pages > 0 ? new PagePool(num_pages) : nullptr; }
NI_HOST_EXPORT void ni_pool_destroy(void* p) { delete static_cast<PagePool*>(p); }
NI_HOST_EXPORT int ni_pool_num_free(void* p) { return static_cast<PagePool*>(p)->num_free(); }
NI_HOST_EXPORT int ni_pool_is_taken(void* p, int page) { return static_cast<PagePool*>(p)->is_taken(page) ? 1 : 0; }
NI_HOST_EXPORT int ni_pool_take(void* p, int n, int32_t* out) { return static_cast<PagePool*>(p)->take(n, out); }
NI_HOST_EXPORT int ni_pool_give_back(void* p, const int32_t* pages, int n) { return static_cast<PagePool*>(p)->give_back(pages, n); }
NI_HOST_EXPORT const char* ni_pool_last_error(void* p) { return static_cast<PagePool*>(p)->error.c_str(); }

// ---- cache manager -------------------------------------------------------------------------------
// windows[g] < 0: the group keeps all keys.
NI_HOST_EXPORT void* ni_cache_create(int n_groups, const int* pages_per_group, const int* windows, int page_size,
                                     int max_requests, int max_tokens_per_request) {
    if (n_groups <= 0 || page_size <= 0 || max_requests <= 0 || max_tokens_per_request <= 0) return nullptr;
    for (int g = 0; g < n_groups; ++g)
        if (pages_per_group[g] <= 0) return nullptr;
    return new CacheManager(n_groups, pages_per_group, windows, page_size, max_requests, max_tokens_per_request);
}
NI_HOST_EXPORT void ni_cache_destroy(void* c) { delete static_cast<CacheManager*>(c); }
NI_HOST_EXPORT const char* ni_cache_last_error(void* c) { return static_cast<CacheManager*>(c)->error.c_str(); }
NI_HOST_EXPORT int ni_cache_table_width(void* c) { return static_cast<CacheManager*>(c)->table_width; }
NI_HOST_EXPORT long long ni_cache_table_version(void* c) { return static_cast<CacheManager*>(c)->table_version; }
NI_HOST_EXPORT int32_t* ni_cache_mirror(void* c, int g) { return static_cast<CacheManager*>(c)->mirror[(size_t)g].data(); }
NI_HOST_EXPORT int ni_cache_has(void* c, long long req) { return static_cast<CacheManager*>(c)->held.count(req) ? 1 : 0; }
NI_HOST_EXPORT int ni_cache_num_free_slots(void* c) { return (int)static_cast<CacheManager*>(c)->free_slots.size(); }
NI_HOST_EXPORT int ni_cache_admit(void* c, long long req) { return static_cast<CacheManager*>(c)->admit(req); }
NI_HOST_EXPORT int ni_cache_slot(void* c, long long req) {
    Held* h = static_cast<CacheManager*>(c)->get(req);
    return h ? h->slot : kErrArgument;
}
NI_HOST_EXPORT int ni_cache_length(void* c, long long req) {
    Held* h = static_cast<CacheManager*>(c)->get(req);
    return h ? h->length : kErrArgument;
}
NI_HOST_EXPORT int ni_cache_pages_needed(void* c, long long req, int n_new, int* out) {
    auto* m = static_cast<CacheManager*>(c);
    Held* h = m->get(req);
    if (!h) return kErrArgument;
    m->pages_needed(*h, n_new, out);
    return kOk;
}
NI_HOST_EXPORT int ni_cache_append(void* c, long long req, int n_new) { return static_cast<CacheManager*>(c)->append(req, n_new); }
// 1 if one more token of the request starts a new page (in every group alike).
NI_HOST_EXPORT int ni_cache_needs_page_for_one(void* c, long long req) {
    auto* m = static_cast<CacheManager*>(c);
    Held* h = m->get(req);
    return h ? (h->length % m->page_size == 0 ? 1 : 0) : kErrArgument;
}
// append(req, 1) for the decode loop: no page arithmetic unless a page starts.
NI_HOST_EXPORT int ni_cache_append_one(void* c, long long req) {
    auto* m = static_cast<CacheManager*>(c);
    Held* h = m->get(req);
    if (!h) return kErrArgument;
    if (h->length % m->page_size == 0 || h->length + 1 > m->max_tokens) return m->append(req, 1);
    h->length += 1;
    return kOk;
}
NI_HOST_EXPORT int ni_cache_release_passed(void* c, long long req) { return static_cast<CacheManager*>(c)->release_passed(req); }
NI_HOST_EXPORT int ni_cache_free(void* c, long long req) { return static_cast<CacheManager*>(c)->free_request(req); }
NI_HOST_EXPORT int ni_cache_check(void* c) { return static_cast<CacheManager*>(c)->check(); }
NI_HOST_EXPORT int ni_cache_pool_num_pages(void* c, int g) { return static_cast<CacheManager*>(c)->pools[(size_t)g].num_pages; }
NI_HOST_EXPORT int ni_cache_pool_num_free(void* c, int g) { return static_cast<CacheManager*>(c)->pools[(size_t)g].num_free(); }
NI_HOST_EXPORT int ni_cache_pool_is_taken(void* c, int g, int page) {
    return static_cast<CacheManager*>(c)->pools[(size_t)g].is_taken(page) ? 1 : 0;
}
// The request's block table of one group (-1 = released); returns its length, copies at most cap entries.
NI_HOST_EXPORT int ni_cache_block_table(void* c, long long req, int g, int32_t* out, int cap) {
    auto* m = static_cast<CacheManager*>(c);
    Held* h = m->get(req);
    if (!h || g < 0 || g >= m->n_groups()) return kErrArgument;
    const auto& t = h->tables[(size_t)g];
    for (int i = 0; i < (int)t.size() && i < cap; ++i) out[i] = t[(size_t)i];
    return (int)t.size();
}

// ---- scheduler -----------------------------------------------------------------------------------
// First come, first served, continuous batching, chunked prefill.  Every step is ONE batch: each
// running request contributes its next tokens - one token if it is decoding, otherwise a portion of
// at most prefill_chunk_size - and waiting requests are admitted in arrival order while the token
// budget, the batch size, the request slots and the pages allow.  Pages are taken portion by
// portion (by the step function; the scheduler only counts them).
//
// When pages run out: the most recently admitted running request is preempted - its pages and slot
// are given back, it returns to the FRONT of the waiting queue and is recomputed later from its
// prompt plus the tokens it had generated.  If the request that needs the page is the only one
// running, the pool is too small for it: it fails and the engine goes on.
//
// The reference admits by batch size and sequence count only, reserves a whole prompt's pages when
// the request is added, runs every prefill portion as a forward pass of its own
// (src/engine/scheduler.cpp:51-91, src/engine/engine.cpp:142-173,215-250) and stops the engine
// when a decode step finds no free page (src/engine/engine.cpp:403-404,194-198).
//
// The scheduler knows requests by id and by counts only; token ids, sampling and stop conditions
// stay with the caller, who reports each sampled token with ni_sched_commit.
namespace {

enum ReqState { kWaiting = 0, kRunning = 1, kFinished = 2, kFailed = 3 };

struct SchedRequest {
    int prompt_len = 0, max_new = 0;
    int n_generated = 0;      // sampled tokens known to the host
    int n_pending = 0;        // sampled tokens still on the device
    int n_computed = 0;       // tokens whose keys/values are in the cache
    int state = kWaiting;
    int n_preempt = 0;
    int remaining() const { return prompt_len + n_generated + n_pending - n_computed; }
};

struct Scheduler {
    CacheManager* cache;
    int max_batch, max_seqs, chunk, token_budget;
    std::deque<long long> waiting;
    std::vector<long long> running;            // in order of admission
    std::unordered_map<long long, SchedRequest> reqs;
    long long n_finished = 0, n_preemptions = 0;
    // the last decision
    std::vector<long long> e_ids, preempted, failed;
    std::vector<int> e_n;
    std::string error;

    void drop(long long id) {
        running.erase(std::remove(running.begin(), running.end(), id), running.end());
        if (cache->held.count(id)) cache->free_request(id);
    }
    void preempt(long long id) {
        drop(id);
        SchedRequest& r = reqs[id];
        r.n_computed = 0;
        r.state = kWaiting;
        ++r.n_preempt;
        ++n_preemptions;
        waiting.push_front(id);
    }
    void fail(long long id) {
        reqs[id].state = kFailed;
        ++n_finished;
        failed.push_back(id);
    }

    void schedule() {
        e_ids.clear(); e_n.clear(); preempted.clear(); failed.clear();
        const int G = cache->n_groups();
        std::vector<int> reserved((size_t)G, 0), need((size_t)G, 0);
        int budget = token_budget;
        int decoding = 0;
        for (long long id : running) decoding += reqs[id].remaining() == 1;
        int portion_budget = std::max(0, budget - decoding);   // decode tokens are set aside first
        auto fits = [&]() {
            for (int g = 0; g < G; ++g)
                if (reserved[(size_t)g] + need[(size_t)g] > cache->pools[(size_t)g].num_free()) return false;
            return true;
        };
        size_t i = 0;
        while (i < running.size()) {
            const long long id = running[i];
            if ((int)e_ids.size() >= max_batch) break;
            const int remaining = reqs[id].remaining();
            const int n = remaining == 1 ? (budget > 0 ? 1 : 0) : std::min(std::min(remaining, chunk), portion_budget);
            if (n <= 0) { ++i; continue; }
            auto it = cache->held.find(id);
            if (it != cache->held.end()) cache->pages_needed(it->second, n, need.data());
            else std::fill(need.begin(), need.end(), (n + cache->page_size - 1) / cache->page_size);
            bool gone = false;
            while (!fits()) {
                const long long victim = running.back();
                if (victim == id) {
                    if (running.size() == 1) {      // alone and still no room: the pool cannot hold this request
                        drop(id);
                        fail(id);
                    } else {
                        preempt(id);
                        preempted.push_back(id);
                    }
                    gone = true;
                    break;
                }
                preempt(victim);
                preempted.push_back(victim);
            }
            if (gone) continue;                      // running[i] is now the next request (or the end)
            e_ids.push_back(id);
            e_n.push_back(n);
            for (int g = 0; g < G; ++g) reserved[(size_t)g] += need[(size_t)g];
            budget -= n;
            if (remaining > 1) portion_budget -= n;
            ++i;
        }
        // admit waiting requests in arrival order; stop at the first that does not fit
        int slots_left = (int)cache->free_slots.size();
        while (!waiting.empty() && preempted.empty() && (int)running.size() < max_seqs &&
               (int)e_ids.size() < max_batch && slots_left > 0) {
            const long long id = waiting.front();
            SchedRequest& r = reqs[id];
            const int n = std::min(std::min(r.remaining(), chunk), portion_budget);
            if (n <= 0) break;
            std::fill(need.begin(), need.end(), (n + cache->page_size - 1) / cache->page_size);
            if (!fits()) {
                if (running.empty() && e_ids.empty()) {   // nothing runs and the first portion still does not fit
                    waiting.pop_front();
                    fail(id);
                    continue;
                }
                break;
            }
            waiting.pop_front();
            r.state = kRunning;
            running.push_back(id);
            e_ids.push_back(id);
            e_n.push_back(n);
            for (int g = 0; g < G; ++g) reserved[(size_t)g] += need[(size_t)g];
            budget -= n;
            portion_budget -= n;
            --slots_left;
        }
    }

    // True if the next decision is known without the tokens of the batch in flight (prev): it held
    // every running request, all of them get their token from it and go on decoding, nobody waits
    // for admission, and every page they need is free.
    bool can_continue(const long long* prev, int n_prev) {
        if (!waiting.empty() || n_prev != (int)running.size()) return false;
        int need = 0;
        for (int i = 0; i < n_prev; ++i) {
            if (prev[i] != running[(size_t)i]) return false;
            const SchedRequest& r = reqs[prev[i]];
            if (r.n_pending != 1 || r.remaining() != 1 || r.n_generated + r.n_pending >= r.max_new) return false;
            auto it = cache->held.find(prev[i]);
            if (it == cache->held.end()) return false;
            need += it->second.length % cache->page_size == 0;
        }
        if ((int)running.size() > std::min(max_batch, token_budget)) return false;
        for (auto& pool : cache->pools)
            if (need > pool.num_free()) return false;
        return true;
    }
};

}  // namespace

NI_HOST_EXPORT void* ni_sched_create(void* cache, int max_batch_size, int max_sequences, int prefill_chunk_size,
                                     int max_num_batched_tokens) {
    if (!cache || max_batch_size <= 0 || max_sequences <= 0 || prefill_chunk_size <= 0 || max_num_batched_tokens <= 0)
        return nullptr;
    auto* s = new Scheduler();
    s->cache = static_cast<CacheManager*>(cache);
    s->max_batch = max_batch_size;
    s->max_seqs = std::min(max_sequences, s->cache->max_requests);
    s->chunk = prefill_chunk_size;
    s->token_budget = max_num_batched_tokens;
    return s;
}
NI_HOST_EXPORT void ni_sched_destroy(void* s) { delete static_cast<Scheduler*>(s); }
NI_HOST_EXPORT int ni_sched_add(void* s, long long id, int prompt_len, int max_new_tokens) {
    auto* sc = static_cast<Scheduler*>(s);
    if (sc->reqs.count(id) || prompt_len <= 0 || max_new_tokens <= 0) return kErrArgument;
    SchedRequest r;
    r.prompt_len = prompt_len;
    r.max_new = max_new_tokens;
    sc->reqs.emplace(id, r);
    sc->waiting.push_back(id);
    return kOk;
}
NI_HOST_EXPORT int ni_sched_has_work(void* s) {
    auto* sc = static_cast<Scheduler*>(s);
    return (!sc->waiting.empty() || !sc->running.empty()) ? 1 : 0;
}
// Decides the next batch.  Returns the number of entries; the decision is read with ni_sched_result.
NI_HOST_EXPORT int ni_sched_schedule(void* s) {
    auto* sc = static_cast<Scheduler*>(s);
    sc->schedule();
    return (int)sc->e_ids.size();
}
// what: 0 = entry ids, 1 = entry token counts, 2 = preempted ids, 3 = failed ids.  Returns the count.
NI_HOST_EXPORT int ni_sched_result(void* s, int what, long long* out, int cap) {
    auto* sc = static_cast<Scheduler*>(s);
    int n = 0;
    auto copy = [&](const std::vector<long long>& v) {
        n = (int)v.size();
        for (int i = 0; i < n && i < cap; ++i) out[i] = v[(size_t)i];
    };
    if (what == 0) copy(sc->e_ids);
    else if (what == 2) copy(sc->preempted);
    else if (what == 3) copy(sc->failed);
    else if (what == 1) {
        n = (int)sc->e_n.size();
        for (int i = 0; i < n && i < cap; ++i) out[i] = sc->e_n[(size_t)i];
    } else return kErrArgument;
    return n;
}
// The batch has been launched: its tokens count as computed, and every emitting request has one
// more sampled token on the way.
NI_HOST_EXPORT int ni_sched_advance(void* s, int n, const long long* ids, const int* counts, int n_emitting,
                                    const long long* emitting) {
    auto* sc = static_cast<Scheduler*>(s);
    for (int i = 0; i < n; ++i) {
        auto it = sc->reqs.find(ids[i]);
        if (it == sc->reqs.end()) return kErrArgument;
        it->second.n_computed += counts[i];
    }
    for (int i = 0; i < n_emitting; ++i) {
        auto it = sc->reqs.find(emitting[i]);
        if (it == sc->reqs.end()) return kErrArgument;
        it->second.n_pending += 1;
    }
    return kOk;
}
// A token on the way has been read.  finished != 0: it ends the request (stop token or length):
// the request leaves the running list (or the waiting queue) and its pages and slot are given back.
NI_HOST_EXPORT int ni_sched_commit(void* s, long long id, int finished) {
    auto* sc = static_cast<Scheduler*>(s);
    auto it = sc->reqs.find(id);
    if (it == sc->reqs.end()) return kErrArgument;
    SchedRequest& r = it->second;
    if (r.state == kFinished || r.state == kFailed || r.n_pending == 0) return kErrArgument;
    r.n_pending -= 1;
    r.n_generated += 1;
    if (finished) {
        if (r.state == kRunning) sc->drop(id);
        else sc->waiting.erase(std::remove(sc->waiting.begin(), sc->waiting.end(), id), sc->waiting.end());
        r.state = kFinished;
        ++sc->n_finished;
    }
    return kOk;
}
// Ends a request in any state as failed (a device error made its cache contents worthless, or the
// caller gives it up): it leaves the running list or the waiting queue, its pages and slot are given
// back, tokens on the way are forgotten.  Returns 1 if it was alive, 0 if it had ended before.
NI_HOST_EXPORT int ni_sched_abort(void* s, long long id) {
    auto* sc = static_cast<Scheduler*>(s);
    auto it = sc->reqs.find(id);
    if (it == sc->reqs.end()) return kErrArgument;
    SchedRequest& r = it->second;
    if (r.state == kFinished || r.state == kFailed) return 0;
    if (r.state == kRunning) sc->drop(id);
    else sc->waiting.erase(std::remove(sc->waiting.begin(), sc->waiting.end(), id), sc->waiting.end());
    r.state = kFailed;
    r.n_pending = 0;
    ++sc->n_finished;
    return 1;
}
NI_HOST_EXPORT int ni_sched_can_continue(void* s, const long long* prev, int n_prev) {
    return static_cast<Scheduler*>(s)->can_continue(prev, n_prev) ? 1 : 0;
}
// field: 0 state, 1 computed tokens, 2 pending tokens, 3 generated tokens, 4 preemptions, 5 remaining.
NI_HOST_EXPORT int ni_sched_get(void* s, long long id, int field) {
    auto* sc = static_cast<Scheduler*>(s);
    auto it = sc->reqs.find(id);
    if (it == sc->reqs.end()) return kErrArgument;
    const SchedRequest& r = it->second;
    switch (field) {
        case 0: return r.state;
        case 1: return r.n_computed;
        case 2: return r.n_pending;
        case 3: return r.n_generated;
        case 4: return r.n_preempt;
        case 5: return r.remaining();
        default: return kErrArgument;
    }
}
// what: 0 running, 1 waiting, 2 finished, 3 total requests, 4 preemptions.
NI_HOST_EXPORT long long ni_sched_stat(void* s, int what) {
    auto* sc = static_cast<Scheduler*>(s);
    switch (what) {
        case 0: return (long long)sc->running.size();
        case 1: return (long long)sc->waiting.size();
        case 2: return sc->n_finished;
        case 3: return (long long)sc->reqs.size();
        case 4: return sc->n_preemptions;
        default: return kErrArgument;
    }
}
