// The host side of a step, natively: the books of cache pages and request slots, and the
// packing of a step's integers into the one buffer that is copied to the device.
//
// What is kept: a page pool per group of cache-owning layers (free list, lowest id first,
// all-or-nothing; page 0 is the null page that is never handed out), a pool of request slots,
// and per live request its slot, its length and one block table per group (logical page ->
// page id). The life of a request is admit -> per step grow, then commit once the step has
// run -> finish; pages that every window has passed go back at commit, everything at finish.
// A page given back twice, or one the pool never handed out, is refused. The same rules as
// tgo_b200/cache/pages.py, which stays as the plain statement of them and is what the tests
// hold this file against (the reference's: internal/prefix/prefix.go:219-226, :343-380,
// internal/prefix/lease.go:66-222, plan.go:160-177).
//
// Requests are named by 64-bit handles that the caller picks. Every call returns a code
// (0: done); what went wrong is told by tgo_cache_last_error. No call throws, allocates
// device memory or touches CUDA.
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <unordered_map>
#include <vector>

#include "host_runtime.h"      // the declarations: a mismatch with a definition below fails to compile

#define TGO_HOST_API extern "C" __attribute__((visibility("default")))

namespace {

enum Code {
    OK = 0,
    PAGES_EXHAUSTED = 1,   // info: group, need, free
    SLOTS_EXHAUSTED = 2,
    ALREADY_LIVE = 3,
    NOT_LIVE = 4,
    BAD_ARGUMENT = 5,
    NO_PAGE = 6,           // a position has no page: info: group, position, entry
    PAGE_MISUSE = 7,       // a page given back twice or not of the pool
    BUFFER_SMALL = 8,      // info[0]: ints needed
    BROKEN_BOOKS = 9,      // check_invariants found a fault
};

constexpr int NULL_PAGE = 0;
constexpr int KIND_FULL = 0, KIND_WINDOW = 1;

struct Pool {
    int num_pages = 0;
    std::vector<int> free_;          // back() is the lowest free id
    std::vector<uint8_t> held;
    long long taken_total = 0, given_total = 0;

    void init(int n) {
        num_pages = n;
        free_.resize(n);
        for (int i = 0; i < n; ++i) free_[i] = n - i;
        held.assign(n + 1, 0);
    }
    int free_count() const { return (int)free_.size(); }
    void take(int n, std::vector<int>& out) {
        for (int i = 0; i < n; ++i) {
            const int p = free_.back();
            free_.pop_back();
            held[p] = 1;
            out.push_back(p);
        }
        taken_total += n;
    }
    // 0, or the page that may not be given
    int give(std::vector<int>& pages) {
        for (int p : pages) {
            if (p < 1 || p > num_pages) return p ? p : -1;
            if (!held[p]) return p;
            held[p] = 0;            // also catches a page named twice in one call
        }
        std::sort(pages.begin(), pages.end(), [](int a, int b) { return a > b; });
        for (int p : pages) free_.push_back(p);
        given_total += (long long)pages.size();
        return 0;
    }
};

struct Request {
    int slot = -1;
    long long length = 0, version = 0;
    std::vector<std::vector<int>> tables;
};

struct Manager {
    std::vector<int> kind, window;
    int page_size = 1;
    std::vector<Pool> pools;
    int num_slots = 0;
    std::vector<int> free_slots;     // back() is the lowest free slot
    std::vector<uint8_t> slot_held;
    std::unordered_map<long long, Request> requests;
    bool has_window = false;
    std::string error;
    long long info[3] = {0, 0, 0};

    int fail(int code, const std::string& what, long long a = 0, long long b = 0, long long c = 0) {
        error = what;
        info[0] = a; info[1] = b; info[2] = c;
        return code;
    }
    long long pages_for(long long tokens) const { return (tokens + page_size - 1) / page_size; }
    long long first_live(int g, long long length) const {
        if (kind[g] == KIND_FULL) return 0;
        return std::max<long long>(0, length - window[g] + 1);
    }
    // logical pages of group g that positions [first live, upto) need and lack
    void missing(const Request& r, int g, long long upto, std::vector<int>& out) const {
        const long long last = pages_for(upto);
        const std::vector<int>& t = r.tables[g];
        if (kind[g] == KIND_FULL) {
            for (long long i = (long long)t.size(); i < last; ++i) out.push_back((int)i);
            return;
        }
        const long long first = first_live(g, r.length) / page_size;
        for (long long i = first; i < last; ++i)
            if (i >= (long long)t.size() || t[i] == NULL_PAGE) out.push_back((int)i);
    }
    int grow(Request& r, long long upto, bool full_only) {
        const int G = (int)kind.size();
        std::vector<std::vector<int>> plan(G);
        for (int g = 0; g < G; ++g) {
            if (full_only && kind[g] != KIND_FULL) continue;
            missing(r, g, upto, plan[g]);
            if ((int)plan[g].size() > pools[g].free_count())
                return fail(PAGES_EXHAUSTED, "cache: group " + std::to_string(g) + " needs " +
                            std::to_string(plan[g].size()) + " more pages and has " +
                            std::to_string(pools[g].free_count()) + " free",
                            g, (long long)plan[g].size(), pools[g].free_count());
        }
        std::vector<int> pages;
        for (int g = 0; g < G; ++g) {
            if (plan[g].empty()) continue;
            pages.clear();
            pools[g].take((int)plan[g].size(), pages);
            std::vector<int>& t = r.tables[g];
            for (size_t j = 0; j < plan[g].size(); ++j) {
                const int i = plan[g][j];
                if ((int)t.size() <= i) t.resize(i + 1, NULL_PAGE);
                t[i] = pages[j];
            }
            ++r.version;
        }
        return OK;
    }
};

Manager* M(void* p) { return (Manager*)p; }

}  // namespace

// kinds[g]: 0 every key, 1 a window of windows[g] keys.
TGO_HOST_API void* tgo_cache_create(int n_groups, const int* kinds, const int* windows, int page_size,
                                    const int* pages_per_group, int num_slots) {
    if (n_groups <= 0 || page_size <= 0 || num_slots <= 0) return nullptr;
    for (int g = 0; g < n_groups; ++g)
        if (pages_per_group[g] <= 0 || (kinds[g] != KIND_FULL && kinds[g] != KIND_WINDOW) ||
            (kinds[g] == KIND_WINDOW && windows[g] <= 0))
            return nullptr;
    Manager* m = new Manager();
    m->kind.assign(kinds, kinds + n_groups);
    m->window.assign(windows, windows + n_groups);
    m->page_size = page_size;
    m->pools.resize(n_groups);
    for (int g = 0; g < n_groups; ++g) {
        m->pools[g].init(pages_per_group[g]);
        m->has_window = m->has_window || kinds[g] == KIND_WINDOW;
    }
    m->num_slots = num_slots;
    m->free_slots.resize(num_slots);
    for (int i = 0; i < num_slots; ++i) m->free_slots[i] = num_slots - 1 - i;
    m->slot_held.assign(num_slots, 0);
    return m;
}

TGO_HOST_API void tgo_cache_destroy(void* p) { delete M(p); }

// The message and the three numbers of the last call that did not return 0.
TGO_HOST_API const char* tgo_cache_last_error(void* p, long long* info) {
    Manager* m = M(p);
    if (info) { info[0] = m->info[0]; info[1] = m->info[1]; info[2] = m->info[2]; }
    return m->error.c_str();
}

// A slot, and pages of the groups that keep every key for `reserve_tokens` positions:
// together or not at all.
TGO_HOST_API int tgo_cache_admit(void* p, long long handle, long long reserve_tokens, int* slot) {
    Manager* m = M(p);
    if (m->requests.count(handle)) return m->fail(ALREADY_LIVE, "cache: the request is already live");
    if (m->free_slots.empty())
        return m->fail(SLOTS_EXHAUSTED, "cache: all " + std::to_string(m->num_slots) + " request slots are taken");
    Request r;
    r.slot = m->free_slots.back();
    r.tables.resize(m->kind.size());
    if (reserve_tokens > 0) {
        const int rc = m->grow(r, reserve_tokens, true);
        if (rc) return rc;                    // nothing was taken: grow plans before it takes
    }
    m->free_slots.pop_back();
    m->slot_held[r.slot] = 1;
    *slot = r.slot;
    m->requests.emplace(handle, std::move(r));
    return OK;
}

// Pages for every position below `upto` that a step may read or write, in all groups or
// in none.
TGO_HOST_API int tgo_cache_grow(void* p, long long handle, long long upto) {
    Manager* m = M(p);
    auto it = m->requests.find(handle);
    if (it == m->requests.end()) return m->fail(NOT_LIVE, "cache: the request is not live");
    Request& r = it->second;
    size_t shortest = r.tables.empty() ? 0 : r.tables[0].size();
    for (const auto& t : r.tables) shortest = std::min(shortest, t.size());
    if (upto <= (long long)shortest * m->page_size) return OK;     // the common decode step
    return m->grow(r, upto, false);
}

// The step landed: the request holds new_length tokens. Pages wholly before the first position
// that a later query can read go back: (group, page) pairs into `released` (as many as fit
// `cap` pairs; *n_released counts all).
TGO_HOST_API int tgo_cache_commit(void* p, long long handle, long long new_length, int* released, int cap,
                                  int* n_released) {
    Manager* m = M(p);
    if (n_released) *n_released = 0;
    auto it = m->requests.find(handle);
    if (it == m->requests.end()) return m->fail(NOT_LIVE, "cache: the request is not live");
    Request& r = it->second;
    if (new_length < r.length) return m->fail(BAD_ARGUMENT, "cache: a request's length cannot shrink");
    r.length = new_length;
    if (!m->has_window) return OK;
    int n = 0;
    std::vector<int> gone;
    for (int g = 0; g < (int)m->kind.size(); ++g) {
        if (m->kind[g] != KIND_WINDOW) continue;
        const long long dead = m->first_live(g, new_length) / m->page_size;
        std::vector<int>& t = r.tables[g];
        gone.clear();
        for (long long i = 0; i < std::min<long long>(dead, (long long)t.size()); ++i)
            if (t[i] != NULL_PAGE) { gone.push_back(t[i]); t[i] = NULL_PAGE; }
        if (gone.empty()) continue;
        for (int pg : gone) {
            if (released && n < cap) { released[2 * n] = g; released[2 * n + 1] = pg; }
            ++n;
        }
        const int bad = m->pools[g].give(gone);
        if (bad) return m->fail(PAGE_MISUSE, "cache: page " + std::to_string(bad) + " cannot be given back", g, bad);
        ++r.version;
    }
    if (n_released) *n_released = n;
    return OK;
}

// Everything the request holds goes back.
TGO_HOST_API int tgo_cache_finish(void* p, long long handle, int* released, int cap, int* n_released) {
    Manager* m = M(p);
    if (n_released) *n_released = 0;
    auto it = m->requests.find(handle);
    if (it == m->requests.end()) return m->fail(NOT_LIVE, "cache: the request is not live");
    Request& r = it->second;
    int n = 0;
    std::vector<int> pages;
    for (int g = 0; g < (int)m->kind.size(); ++g) {
        pages.clear();
        for (int pg : r.tables[g])
            if (pg != NULL_PAGE) pages.push_back(pg);
        for (int pg : pages) {
            if (released && n < cap) { released[2 * n] = g; released[2 * n + 1] = pg; }
            ++n;
        }
        if (!pages.empty()) {
            const int bad = m->pools[g].give(pages);
            if (bad) return m->fail(PAGE_MISUSE, "cache: page " + std::to_string(bad) + " cannot be given back", g, bad);
        }
    }
    m->slot_held[r.slot] = 0;
    m->free_slots.push_back(r.slot);
    std::sort(m->free_slots.begin(), m->free_slots.end(), [](int a, int b) { return a > b; });
    m->requests.erase(it);
    if (n_released) *n_released = n;
    return OK;
}

// ---------------------------------------------------------------------------- queries
// what: 0 length, 1 slot, 2 version, 3 live (1/0); for 0-2 the request must be live (-1 else).
TGO_HOST_API long long tgo_cache_request(void* p, long long handle, int what) {
    Manager* m = M(p);
    auto it = m->requests.find(handle);
    if (what == 3) return it != m->requests.end();
    if (it == m->requests.end()) return -1;
    return what == 0 ? it->second.length : what == 1 ? it->second.slot : it->second.version;
}

// The block table of a group: its length; the first `cap` entries into `out`.
TGO_HOST_API int tgo_cache_table(void* p, long long handle, int group, int* out, int cap) {
    Manager* m = M(p);
    auto it = m->requests.find(handle);
    if (it == m->requests.end() || group < 0 || group >= (int)m->kind.size()) return -1;
    const std::vector<int>& t = it->second.tables[group];
    for (int i = 0; i < (int)t.size() && i < cap; ++i) out[i] = t[i];
    return (int)t.size();
}

// what: 0 free pages, 1 held pages, 2 pages in all, 3 taken in all so far, 4 given back so far.
TGO_HOST_API long long tgo_cache_pool(void* p, int group, int what) {
    Manager* m = M(p);
    if (group < 0 || group >= (int)m->pools.size()) return -1;
    const Pool& pool = m->pools[group];
    switch (what) {
        case 0: return pool.free_count();
        case 1: return pool.num_pages - pool.free_count();
        case 2: return pool.num_pages;
        case 3: return pool.taken_total;
        default: return pool.given_total;
    }
}
TGO_HOST_API int tgo_cache_page_is_held(void* p, int group, int page) {
    Manager* m = M(p);
    if (group < 0 || group >= (int)m->pools.size()) return 0;
    return page >= 1 && page <= m->pools[group].num_pages && m->pools[group].held[page];
}
TGO_HOST_API int tgo_cache_free_slots(void* p) { return (int)M(p)->free_slots.size(); }
TGO_HOST_API int tgo_cache_live_requests(void* p) { return (int)M(p)->requests.size(); }

// Could a request of this many tokens ever fit, with the pools empty, when it is run in steps
// of at most step_tokens tokens? A window group gives pages back only when a step has landed,
// so during a step it holds the window and the step's own tokens.
TGO_HOST_API int tgo_cache_can_hold(void* p, long long n_tokens, long long step_tokens) {
    Manager* m = M(p);
    if (step_tokens < 1) step_tokens = 1;
    for (int g = 0; g < (int)m->kind.size(); ++g) {
        long long need = m->pages_for(n_tokens);
        if (m->kind[g] == KIND_WINDOW)
            need = std::min(need, m->pages_for(m->window[g] - 1 + step_tokens) + 1);
        if (need > m->pools[g].num_pages) return 0;
    }
    return 1;
}

// Row of the paged storage that holds `position`, or -1 (no page there: see last_error).
TGO_HOST_API long long tgo_cache_slot_of(void* p, long long handle, int group, long long position) {
    Manager* m = M(p);
    auto it = m->requests.find(handle);
    if (it == m->requests.end() || group < 0 || group >= (int)m->kind.size() || position < 0) {
        m->fail(NOT_LIVE, "cache: the request is not live");
        return -1;
    }
    const std::vector<int>& t = it->second.tables[group];
    const long long i = position / m->page_size;
    if (i >= (long long)t.size() || t[i] == NULL_PAGE) {
        m->fail(NO_PAGE, "cache: position " + std::to_string(position) + " has no page in group " +
                std::to_string(group), group, position);
        return -1;
    }
    return (long long)t[i] * m->page_size + position % m->page_size;
}

// No page lost, none held twice: every pool's held pages are exactly the pages in the live
// requests' tables, and no two requests share a slot.
TGO_HOST_API int tgo_cache_check(void* p) {
    Manager* m = M(p);
    for (int g = 0; g < (int)m->pools.size(); ++g) {
        const Pool& pool = m->pools[g];
        std::vector<uint8_t> seen(pool.num_pages + 1, 0);
        long long n = 0;
        for (const auto& kv : m->requests)
            for (int pg : kv.second.tables[g]) {
                if (pg == NULL_PAGE) continue;
                if (pg < 1 || pg > pool.num_pages || !pool.held[pg])
                    return m->fail(BROKEN_BOOKS, "cache: group " + std::to_string(g) + " table names free page " + std::to_string(pg));
                if (seen[pg])
                    return m->fail(BROKEN_BOOKS, "cache: group " + std::to_string(g) + " has a page in two tables");
                seen[pg] = 1;
                ++n;
            }
        if (n != pool.num_pages - pool.free_count())
            return m->fail(BROKEN_BOOKS, "cache: group " + std::to_string(g) + " holds " +
                           std::to_string(pool.num_pages - pool.free_count()) + " pages and the tables name " + std::to_string(n));
    }
    std::vector<uint8_t> slots(m->num_slots, 0);
    for (const auto& kv : m->requests) {
        const int s = kv.second.slot;
        if (s < 0 || s >= m->num_slots || slots[s]) return m->fail(BROKEN_BOOKS, "cache: two requests share a slot");
        slots[s] = 1;
    }
    return OK;
}

// ------------------------------------------------------------------------------ a step
// Pages for what the step's requests are about to write: request by request, each in all its
// groups or not at all. On a refusal the requests before the refused one keep what they got
// (they would ask for the same pages again) and info[] tells group, need and free;
// *refused is the entry that was refused. *widest: the longest block table among the
// requests afterwards (what decides which captured graph the step runs through).
TGO_HOST_API int tgo_step_grow(void* p, int n, const long long* handles, const int* extents, int* refused,
                              int* widest) {
    Manager* m = M(p);
    if (widest) *widest = 0;
    for (int i = 0; i < n; ++i) {
        auto it = m->requests.find(handles[i]);
        if (it == m->requests.end()) {
            if (refused) *refused = i;
            return m->fail(NOT_LIVE, "cache: the request is not live");
        }
        const int rc = tgo_cache_grow(p, handles[i], it->second.length + extents[i]);
        if (rc) {
            if (refused) *refused = i;
            return rc;
        }
        if (widest)
            for (const auto& t : it->second.tables) *widest = std::max(*widest, (int)t.size());
    }
    return OK;
}

// The step has run: every request's length moves on by what it brought, and pages that
// every window has passed go back.
TGO_HOST_API int tgo_step_commit(void* p, int n, const long long* handles, const int* extents) {
    Manager* m = M(p);
    for (int i = 0; i < n; ++i) {
        auto it = m->requests.find(handles[i]);
        if (it == m->requests.end()) return m->fail(NOT_LIVE, "cache: the request is not live");
        const int rc = tgo_cache_commit(p, handles[i], it->second.length + extents[i], nullptr, 0, nullptr);
        if (rc) return rc;
    }
    return OK;
}

// The integers of one step as one flat int32 array, the layout the device side reads:
//   ids[T] pos[T] seq[T] q_start[B+1] ctx[B] state_slot[B] rows[n_rows]
//   then per group: slots[T] table[B * width]
// T tokens of B requests. With pad_to > n, requests that bring nothing fill the batch: one
// token each at position -1, context 0, the spare state slot (num_slots), cache row -1. A
// group's table is as wide as the longest table among the step's requests, rounded up to
// width_quantum, padded with the null page. rows: the wanted places as token indices
// (want_flat holds them per entry, relative to the entry's first token), or every token
// (all_rows).
// meta: [T, B, n_rows, largest context, ints written, width of each group..., then the
// length before the step of each entry...]: 5 + groups + n ints.
// Returns BUFFER_SMALL with info[0] = ints needed if `cap` is too small.
TGO_HOST_API int tgo_step_pack(void* p, int n, const long long* handles, const int* extents,
                               const int* tokens_flat, const int* n_want, const int* want_flat, int pad_to,
                               int width_quantum, int all_rows, int32_t* out, long long cap, int* meta) {
    Manager* m = M(p);
    const int G = (int)m->kind.size();
    if (n <= 0 || width_quantum <= 0) return m->fail(BAD_ARGUMENT, "step: an empty batch carries nothing");
    std::vector<const Request*> reqs(n);
    long long n_tok = 0, n_rows = 0;
    for (int i = 0; i < n; ++i) {
        auto it = m->requests.find(handles[i]);
        if (it == m->requests.end()) return m->fail(NOT_LIVE, "cache: the request is not live", i);
        reqs[i] = &it->second;
        if (extents[i] <= 0) return m->fail(BAD_ARGUMENT, "step: a request brings no tokens", i);
        n_tok += extents[i];
        n_rows += n_want[i];
    }
    const int n_pad = pad_to > n ? pad_to - n : 0;
    const long long B = n + n_pad, T = n_tok + n_pad;
    if (all_rows) n_rows = T;
    std::vector<long long> widths(G);
    long long total = 3 * T + (B + 1) + 2 * B + n_rows;
    for (int g = 0; g < G; ++g) {
        long long w = 1;
        for (int i = 0; i < n; ++i) w = std::max<long long>(w, (long long)reqs[i]->tables[g].size());
        widths[g] = (w + width_quantum - 1) / width_quantum * width_quantum;
        total += T + B * widths[g];
    }
    if (total > cap || !out) return m->fail(BUFFER_SMALL, "step: the buffer is too small", total);
    int32_t* ids = out;
    int32_t* pos = out + T;
    int32_t* seq = out + 2 * T;
    int32_t* q_start = out + 3 * T;
    int32_t* ctx = q_start + B + 1;
    int32_t* st_slot = ctx + B;
    int32_t* rows = st_slot + B;
    int32_t* rest = rows + n_rows;
    long long at = 0, row_at = 0, want_at = 0, max_ctx = 0;
    for (int i = 0; i < n; ++i) {
        const long long first = reqs[i]->length;
        q_start[i] = (int32_t)at;
        for (int j = 0; j < extents[i]; ++j) {
            ids[at + j] = tokens_flat[at + j];
            pos[at + j] = (int32_t)(first + j);
            seq[at + j] = i;
        }
        if (!all_rows)
            for (int j = 0; j < n_want[i]; ++j) {
                const int wv = want_flat[want_at + j];
                if (wv < 0 || wv >= extents[i]) return m->fail(BAD_ARGUMENT, "step: a wanted place lies outside the request's tokens", i, wv);
                rows[row_at++] = (int32_t)(at + wv);
            }
        want_at += n_want[i];
        ctx[i] = (int32_t)(first + extents[i]);
        max_ctx = std::max<long long>(max_ctx, first + extents[i]);
        st_slot[i] = reqs[i]->slot;
        meta[5 + G + i] = (int)first;
        at += extents[i];
    }
    q_start[n] = (int32_t)at;
    for (int j = 0; j < n_pad; ++j) {
        ids[n_tok + j] = 0;
        pos[n_tok + j] = -1;
        seq[n_tok + j] = n + j;
        q_start[n + 1 + j] = (int32_t)(n_tok + 1 + j);
        ctx[n + j] = 0;
        st_slot[n + j] = m->num_slots;
    }
    if (all_rows)
        for (long long j = 0; j < T; ++j) rows[j] = (int32_t)j;
    const int ps = m->page_size;
    for (int g = 0; g < G; ++g) {
        int32_t* slots = rest;
        int32_t* table = rest + T;
        rest = table + B * widths[g];
        const long long w = widths[g];
        for (long long b = 0; b < B; ++b) {
            int32_t* row = table + b * w;
            long long have = 0;
            if (b < n) {
                const std::vector<int>& t = reqs[b]->tables[g];
                have = (long long)t.size();
                for (long long j = 0; j < have; ++j) row[j] = t[j];
            }
            for (long long j = have; j < w; ++j) row[j] = NULL_PAGE;
        }
        for (long long j = 0; j < n_tok; ++j) {
            const long long b = seq[j], ps_i = pos[j] / ps;
            const int32_t page = ps_i < w ? table[b * w + ps_i] : NULL_PAGE;
            if (page == NULL_PAGE)
                return m->fail(NO_PAGE, "cache: position " + std::to_string(pos[j]) + " has no page in group " +
                               std::to_string(g), g, pos[j], b);
            slots[j] = (int32_t)((long long)page * ps + pos[j] % ps);
        }
        for (long long j = n_tok; j < T; ++j) slots[j] = -1;
        meta[5 + g] = (int)w;
    }
    meta[0] = (int)T; meta[1] = (int)B; meta[2] = (int)n_rows; meta[3] = (int)max_ctx; meta[4] = (int)total;
    return OK;
}

// The longest block table among the step's requests, over all groups (what decides which
// captured graph a step runs through).
TGO_HOST_API int tgo_step_widest_table(void* p, int n, const long long* handles) {
    Manager* m = M(p);
    size_t widest = 0;
    for (int i = 0; i < n; ++i) {
        auto it = m->requests.find(handles[i]);
        if (it == m->requests.end()) return -1;
        for (const auto& t : it->second.tables) widest = std::max(widest, t.size());
    }
    return (int)widest;
}

// ---------------------------------------------------------------------- the scheduler's policy
// Which slots the next step carries and how many tokens of each (schedule.go:80-150 is the
// reference's; the budget here is a real limit on a step's tokens). Pass 1: every live slot
// still in its prompt brings min(chunk, what is left of its prompt, what is left of the
// budget), in slot order, after one token has been set aside for every decoding slot. Pass 2:
// every slot past its prompt brings its one fed token. Per slot i: live[i], prompt_len[i]
// (prompt and fed tokens), prefilled[i] (how many of them have run), has_feed[i]. The work
// comes back in slot order: out_slot, out_count, out_prefill (1: prompt tokens starting at
// prefilled[slot]; 0: the fed token). Returns the number of work items, or -1 for a chunk or
// budget that is not positive.
TGO_HOST_API int tgo_schedule_next_step(int n_slots, const int* live, const long long* prompt_len,
                                        const long long* prefilled, const int* has_feed, long long chunk,
                                        long long budget, int* out_slot, long long* out_count, int* out_prefill) {
    if (chunk <= 0 || budget <= 0) return -1;
    long long decoders = 0;
    for (int i = 0; i < n_slots; ++i)
        if (live[i] && prefilled[i] >= prompt_len[i] && has_feed[i]) ++decoders;
    long long left = std::max<long long>(budget - decoders, 0);
    std::vector<long long> count(n_slots, 0);
    std::vector<int> is_prefill(n_slots, 0);
    for (int i = 0; i < n_slots; ++i) {
        if (!live[i] || prefilled[i] >= prompt_len[i]) continue;
        const long long n = std::min(std::min(chunk, prompt_len[i] - prefilled[i]), left);
        if (n <= 0) continue;
        count[i] = n;
        is_prefill[i] = 1;
        left -= n;
    }
    left += std::min(decoders, budget);
    for (int i = 0; i < n_slots; ++i) {
        if (!live[i] || prefilled[i] < prompt_len[i] || !has_feed[i] || left <= 0) continue;
        count[i] = 1;
        left -= 1;
    }
    int n_work = 0;
    for (int i = 0; i < n_slots; ++i)
        if (count[i] > 0) {
            out_slot[n_work] = i;
            out_count[n_work] = count[i];
            out_prefill[n_work] = is_prefill[i];
            ++n_work;
        }
    return n_work;
}

// The slot to evict when pages run out: the latest arrival, one still in its prompt before
// any that decodes (it has the least work to lose). -1 if none is live.
TGO_HOST_API int tgo_schedule_victim(int n_slots, const int* live, const int* in_prompt, const long long* arrived) {
    int best = -1;
    for (int i = 0; i < n_slots; ++i) {
        if (!live[i]) continue;
        if (best < 0 || in_prompt[i] > in_prompt[best] ||
            (in_prompt[i] == in_prompt[best] && arrived[i] > arrived[best]))
            best = i;
    }
    return best;
}
