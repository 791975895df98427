// The host side of the engine that runs at every step, in C++: page pools, state slots, the block tables of
// the requests, and the packing of one step's batch tables into the pinned buffers the kernels read.
//
// Plain C++17 with a C interface (no CUDA, no Python headers): built into a library of its own and loaded with
// ctypes, so the bookkeeping is testable on a machine without a GPU. The Python classes of `cache/` and
// `engine/batch.py` are thin faces of what is here; they own the names of requests (any hashable value there, a
// 64-bit handle here), the device memory and the choice of groups.
//
// The rules are the reference's (docs/24-paged-kv-cache.md:57-72, src/main/java/org/robomiri/jllm/kv/KvPool.java:
// 249-275, kv/KvSequence.java:116-157): a page is `page_size` consecutive positions of every layer run of a group;
// position p of a request lives in page table[p / page_size], row p % page_size; the pool hands out the page
// freed last first; `reserve` takes all the pages a step needs or none; a windowed group gives a page back once no
// later query can see it (its table entry becomes -1); `close` gives everything back. Errors come back as a code
// and a text (`jh_last_error`): 1 = a wrong argument, 2 = no free page or slot, 3 = the books do not add up (a
// bug), 4 = no such request.
#include <algorithm>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <string>
#include <unordered_map>
#include <vector>

#define JH_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

enum { JH_OK = 0, JH_VALUE = 1, JH_EXHAUSTED = 2, JH_BOOKKEEPING = 3, JH_KEY = 4 };
constexpr int RELEASED = -1;
constexpr long long NOBODY = INT64_MIN;

thread_local std::string g_error;

int fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_error = buf;
    return code;
}

// ---- a pool of ids (pages, or state slots) with one holder each ------------------------------------------------
struct Pool {
    int n = 0;
    std::string name;
    std::vector<int> free_list;          // back() goes out next: id 0 first, then whatever was freed last
    std::vector<long long> holder;
    std::vector<char> used_before;
    long long allocations = 0, reuses = 0;

    void init(int count, const std::string& nm) {
        n = count;
        name = nm;
        free_list.resize(count);
        for (int i = 0; i < count; ++i) free_list[i] = count - 1 - i;
        holder.assign(count, NOBODY);
        used_before.assign(count, 0);
    }
    int num_free() const { return (int)free_list.size(); }
    int alloc(long long who, int* out) {
        if (who == NOBODY) return fail(JH_VALUE, "a page needs a holder");
        if (free_list.empty()) return fail(JH_EXHAUSTED, "%s: all %d are held", name.c_str(), n);
        const int id = free_list.back();
        free_list.pop_back();
        if (holder[id] != NOBODY)
            return fail(JH_BOOKKEEPING, "%s: %d is free and held by #%lld", name.c_str(), id, holder[id]);
        holder[id] = who;
        ++allocations;
        if (used_before[id]) ++reuses;
        used_before[id] = 1;
        *out = id;
        return JH_OK;
    }
    int release(int id, long long who) {
        if (id < 0 || id >= n) return fail(JH_BOOKKEEPING, "%s: %d does not exist", name.c_str(), id);
        if (holder[id] == NOBODY) return fail(JH_BOOKKEEPING, "%s: %d is freed twice", name.c_str(), id);
        if (holder[id] != who)
            return fail(JH_BOOKKEEPING, "%s: %d is held by #%lld, freed by #%lld", name.c_str(), id, holder[id], who);
        holder[id] = NOBODY;
        free_list.push_back(id);
        return JH_OK;
    }
    int check() const {   // every id is either free once or held once
        std::vector<char> is_free(n, 0);
        for (int id : free_list) {
            if (id < 0 || id >= n || is_free[id]) return fail(JH_BOOKKEEPING, "%s: %d is on the free list twice", name.c_str(), id);
            is_free[id] = 1;
        }
        for (int id = 0; id < n; ++id)
            if ((is_free[id] != 0) == (holder[id] != NOBODY))
                return fail(JH_BOOKKEEPING, "%s: %d is %s", name.c_str(), id, is_free[id] ? "free and held" : "lost");
        return JH_OK;
    }
};

// ---- the cache's books ---------------------------------------------------------------------------------------------
struct Request {
    int slot = -1, length = 0;
    long long epoch = 0;
    std::vector<std::vector<int>> tables;   // one per paged group
};

struct Cache {
    int page_size = 1, num_pages = 0;
    std::vector<int> windows;               // per paged group; 0 = every earlier position
    std::vector<Pool> pools;
    Pool slots;
    std::unordered_map<long long, Request> requests;
    long long next_epoch = 1;

    int pages_for(int positions) const { return (positions + page_size - 1) / page_size; }
    int first_needed_page(int g, int length) const {   // pages below hold only positions no later query can see
        if (windows[g] <= 0) return 0;
        return std::max(0, length + 1 - windows[g]) / page_size;
    }
    Request* find(long long id) {
        auto it = requests.find(id);
        return it == requests.end() ? nullptr : &it->second;
    }
    void drop_tail(long long id, Request& r, int keep) {
        for (size_t g = 0; g < pools.size(); ++g) {
            auto& table = r.tables[g];
            while ((int)table.size() > keep) {
                const int page = table.back();
                table.pop_back();
                if (page != RELEASED) pools[g].release(page, id);
            }
        }
    }
    int truncate(long long id, Request& r, int length) {
        if (length >= r.length) return JH_OK;
        const int keep = pages_for(length);
        for (size_t g = 0; g < pools.size(); ++g) {   // first look, then touch: a refused rewind changes nothing
            if (windows[g] > 0 && first_needed_page((int)g, r.length) > first_needed_page((int)g, length)) {
                const auto& table = r.tables[g];
                for (int i = first_needed_page((int)g, length); i < keep && i < (int)table.size(); ++i)
                    if (table[i] == RELEASED)
                        return fail(JH_VALUE, "request #%lld: a windowed group has released pages that a rewind to %d needs; "
                                              "recompute from the start", id, length);
            }
        }
        r.epoch = next_epoch++;
        drop_tail(id, r, keep);
        r.length = length;
        return JH_OK;
    }
    int reserve(long long id, int start, int n) {
        Request* r = find(id);
        if (!r) return fail(JH_KEY, "request #%lld is not open", id);
        if (start < 0 || n < 1) return fail(JH_VALUE, "reserve: start=%d n=%d", start, n);
        if (start > r->length)
            return fail(JH_VALUE, "request #%lld holds %d positions, a step cannot start at %d", id, r->length, start);
        if (start < r->length) {
            const int rc = truncate(id, *r, start);
            if (rc != JH_OK) return rc;
        }
        const int want = pages_for(start + n);
        std::vector<std::pair<int, int>> taken;
        for (size_t g = 0; g < pools.size(); ++g) {
            auto& table = r->tables[g];
            while ((int)table.size() < want) {
                int page = -1;
                const int rc = pools[g].alloc(id, &page);
                if (rc != JH_OK) {   // all or nothing: give back what this call took
                    const std::string why = g_error;
                    r->epoch = next_epoch++;
                    for (auto it = taken.rbegin(); it != taken.rend(); ++it) {
                        auto& t = r->tables[it->first];
                        if (t.empty() || t.back() != it->second)
                            return fail(JH_BOOKKEEPING, "rollback of a failed reserve lost track of a page");
                        t.pop_back();
                        pools[it->first].release(it->second, id);
                    }
                    g_error = why;
                    return rc;
                }
                table.push_back(page);
                taken.emplace_back((int)g, page);
            }
        }
        return JH_OK;
    }
    // The request now holds `length` positions; (group, page) pairs a window has passed go to `released`.
    int commit(long long id, int length, std::vector<int>* released) {
        Request* r = find(id);
        if (!r) return fail(JH_KEY, "request #%lld is not open", id);
        if (length < r->length)
            return fail(JH_VALUE, "commit cannot shorten a request (%d -> %d); use truncate", r->length, length);
        r->length = length;
        bool any = false;
        for (size_t g = 0; g < pools.size(); ++g) {
            auto& table = r->tables[g];
            if ((long long)length > (long long)table.size() * page_size)
                return fail(JH_BOOKKEEPING, "request #%lld committed %d positions beyond its pages", id, length);
            const int upto = std::min(first_needed_page((int)g, length), (int)table.size());
            for (int i = 0; i < upto; ++i) {
                if (table[i] == RELEASED) continue;
                const int rc = pools[g].release(table[i], id);
                if (rc != JH_OK) return rc;
                if (released) {
                    released->push_back((int)g);
                    released->push_back(table[i]);
                }
                table[i] = RELEASED;
                any = true;
            }
        }
        if (any) r->epoch = next_epoch++;
        return JH_OK;
    }
    int trim(long long id) {
        Request* r = find(id);
        if (!r) return fail(JH_KEY, "request #%lld is not open", id);
        r->epoch = next_epoch++;
        drop_tail(id, *r, pages_for(r->length));
        return JH_OK;
    }
    int check() const {
        int rc = slots.check();
        if (rc != JH_OK) return rc;
        for (size_t g = 0; g < pools.size(); ++g) {
            rc = pools[g].check();
            if (rc != JH_OK) return rc;
            std::unordered_map<int, long long> seen;
            for (const auto& kv : requests) {
                for (int page : kv.second.tables[g]) {
                    if (page == RELEASED) continue;
                    auto it = seen.find(page);
                    if (it != seen.end())
                        return fail(JH_BOOKKEEPING, "group %d: page %d is in the tables of #%lld and #%lld", (int)g, page,
                                    it->second, kv.first);
                    seen[page] = kv.first;
                    if (pools[g].holder[page] != kv.first)
                        return fail(JH_BOOKKEEPING, "group %d: page %d is in the table of #%lld but held by #%lld", (int)g,
                                    page, kv.first, pools[g].holder[page]);
                }
            }
            const int held = pools[g].n - pools[g].num_free();
            if ((int)seen.size() != held)
                return fail(JH_BOOKKEEPING, "group %d: %d pages are held, %d are in tables", (int)g, held, (int)seen.size());
        }
        return JH_OK;
    }
};

// ---- one step's tables ---------------------------------------------------------------------------------------------
// What each row of the host block tables holds, so that a row is only extended while nothing else about the
// request's table changed (its epoch).
struct Builder {
    int max_rows, max_segments, max_blocks, groups, page_size;
    struct Held {
        long long request = NOBODY, epoch = 0;
        int entries = 0;
    };
    std::vector<Held> rows;   // [groups][max_segments]
};

}  // namespace

JH_EXPORT const char* jh_last_error() { return g_error.c_str(); }

// ---- stand-alone pools (the Python classes PagePool and StateSlotPool) ------------------------------------------------
JH_EXPORT void* jh_pool_new(int count, const char* name) {
    if (count < 1) {
        fail(JH_VALUE, "a pool needs at least one entry, got %d", count);
        return nullptr;
    }
    Pool* p = new Pool();
    p->init(count, name ? name : "pool");
    return p;
}
JH_EXPORT void jh_pool_delete(void* p) { delete static_cast<Pool*>(p); }
JH_EXPORT int jh_pool_alloc(void* p, long long who, int* out) { return static_cast<Pool*>(p)->alloc(who, out); }
JH_EXPORT int jh_pool_free(void* p, int id, long long who) { return static_cast<Pool*>(p)->release(id, who); }
JH_EXPORT int jh_pool_check(void* p) { return static_cast<Pool*>(p)->check(); }
JH_EXPORT int jh_pool_num_free(void* p) { return static_cast<Pool*>(p)->num_free(); }
JH_EXPORT long long jh_pool_holder(void* p, int id) {
    Pool* pool = static_cast<Pool*>(p);
    return id >= 0 && id < pool->n ? pool->holder[id] : NOBODY;
}
JH_EXPORT void jh_pool_stats(void* p, long long* allocations, long long* reuses) {
    *allocations = static_cast<Pool*>(p)->allocations;
    *reuses = static_cast<Pool*>(p)->reuses;
}

// ---- the cache ---------------------------------------------------------------------------------------------------------
JH_EXPORT void* jh_cache_new(int groups, const int* windows, int page_size, int num_pages, int max_requests) {
    if (page_size < 1 || num_pages < 1 || max_requests < 1 || groups < 0) {
        fail(JH_VALUE, "cache: page_size=%d num_pages=%d max_requests=%d groups=%d", page_size, num_pages, max_requests, groups);
        return nullptr;
    }
    Cache* c = new Cache();
    c->page_size = page_size;
    c->num_pages = num_pages;
    c->windows.assign(windows, windows + groups);
    c->pools.resize(groups);
    for (int g = 0; g < groups; ++g) c->pools[g].init(num_pages, "group" + std::to_string(g) + " pages");
    c->slots.init(max_requests, "state slots");
    return c;
}
JH_EXPORT void jh_cache_delete(void* c) { delete static_cast<Cache*>(c); }

JH_EXPORT int jh_cache_open(void* cv, long long id, int* slot_out) {
    Cache* c = static_cast<Cache*>(cv);
    if (c->find(id)) return fail(JH_VALUE, "request #%lld is open already", id);
    int slot = -1;
    const int rc = c->slots.alloc(id, &slot);
    if (rc != JH_OK) return rc;
    Request r;
    r.slot = slot;
    r.epoch = c->next_epoch++;
    r.tables.resize(c->pools.size());
    c->requests.emplace(id, std::move(r));
    if (slot_out) *slot_out = slot;
    return JH_OK;
}
JH_EXPORT int jh_cache_close(void* cv, long long id) {
    Cache* c = static_cast<Cache*>(cv);
    Request* r = c->find(id);
    if (!r) return fail(JH_KEY, "request #%lld is not open", id);
    c->drop_tail(id, *r, 0);
    const int rc = c->slots.release(r->slot, id);
    c->requests.erase(id);
    return rc;
}
JH_EXPORT int jh_cache_is_open(void* cv, long long id) { return static_cast<Cache*>(cv)->find(id) != nullptr; }
JH_EXPORT int jh_cache_num_requests(void* cv) { return (int)static_cast<Cache*>(cv)->requests.size(); }
JH_EXPORT int jh_cache_request_ids(void* cv, long long* out, int cap) {
    Cache* c = static_cast<Cache*>(cv);
    int i = 0;
    for (const auto& kv : c->requests)
        if (i < cap) out[i++] = kv.first;
    return i;
}
// length, state slot, epoch and the number of table entries per group (`entries` may be null)
JH_EXPORT int jh_cache_request(void* cv, long long id, int* length, int* slot, long long* epoch, int* entries) {
    Cache* c = static_cast<Cache*>(cv);
    Request* r = c->find(id);
    if (!r) return fail(JH_KEY, "request #%lld is not open", id);
    *length = r->length;
    *slot = r->slot;
    *epoch = r->epoch;
    if (entries)
        for (size_t g = 0; g < r->tables.size(); ++g) entries[g] = (int)r->tables[g].size();
    return JH_OK;
}
JH_EXPORT int jh_cache_table(void* cv, long long id, int group, int* out, int cap) {
    Cache* c = static_cast<Cache*>(cv);
    Request* r = c->find(id);
    if (!r) return fail(JH_KEY, "request #%lld is not open", id);
    if (group < 0 || group >= (int)r->tables.size()) return fail(JH_VALUE, "no paged group %d", group);
    const auto& t = r->tables[group];
    if ((int)t.size() > cap) return fail(JH_VALUE, "table of %d entries, room for %d", (int)t.size(), cap);
    std::copy(t.begin(), t.end(), out);
    return JH_OK;
}
JH_EXPORT int jh_cache_pages_missing(void* cv, long long id, int start, int n, int* out) {
    Cache* c = static_cast<Cache*>(cv);
    Request* r = c->find(id);
    for (size_t g = 0; g < c->pools.size(); ++g) {
        int have = r ? (int)r->tables[g].size() : 0;
        if (r && start < r->length) have = std::min(have, c->pages_for(start));
        out[g] = std::max(0, c->pages_for(start + n) - have);
    }
    return JH_OK;
}
JH_EXPORT int jh_cache_can_reserve(void* cv, long long id, int start, int n) {
    Cache* c = static_cast<Cache*>(cv);
    std::vector<int> missing(c->pools.size());
    jh_cache_pages_missing(cv, id, start, n, missing.data());
    for (size_t g = 0; g < c->pools.size(); ++g)
        if (missing[g] > c->pools[g].num_free()) return 0;
    return 1;
}
JH_EXPORT int jh_cache_reserve(void* cv, long long id, int start, int n) { return static_cast<Cache*>(cv)->reserve(id, start, n); }
// `released` receives (group, page) pairs, at most cap / 2 of them; *count = pairs that were released in all
JH_EXPORT int jh_cache_commit(void* cv, long long id, int length, int* released, int cap, int* count) {
    std::vector<int> pairs;
    const int rc = static_cast<Cache*>(cv)->commit(id, length, &pairs);
    if (count) *count = (int)pairs.size() / 2;
    if (released) std::copy(pairs.begin(), pairs.begin() + std::min((int)pairs.size(), cap), released);
    return rc;
}
JH_EXPORT int jh_cache_truncate(void* cv, long long id, int length) {
    Cache* c = static_cast<Cache*>(cv);
    Request* r = c->find(id);
    if (!r) return fail(JH_KEY, "request #%lld is not open", id);
    return c->truncate(id, *r, length);
}
JH_EXPORT int jh_cache_trim(void* cv, long long id) { return static_cast<Cache*>(cv)->trim(id); }
JH_EXPORT int jh_cache_check(void* cv) { return static_cast<Cache*>(cv)->check(); }
JH_EXPORT int jh_cache_free_pages(void* cv, int* out) {
    Cache* c = static_cast<Cache*>(cv);
    for (size_t g = 0; g < c->pools.size(); ++g) out[g] = c->pools[g].num_free();
    return JH_OK;
}
JH_EXPORT void* jh_cache_pool(void* cv, int group) {   // a view for jh_pool_* reads; -1 = the state slots
    Cache* c = static_cast<Cache*>(cv);
    if (group < 0) return &c->slots;
    return group < (int)c->pools.size() ? &c->pools[group] : nullptr;
}

// ---- a step: reserve for every segment (all or none), and commit after it ran --------------------------------------------
JH_EXPORT int jh_step_reserve(void* cv, int segments, const long long* ids, const int* starts, const int* counts) {
    Cache* c = static_cast<Cache*>(cv);
    for (int i = 0; i < segments; ++i) {
        const int rc = c->reserve(ids[i], starts[i], counts[i]);
        if (rc != JH_OK) {
            const std::string why = g_error;
            for (int j = 0; j < i; ++j) c->trim(ids[j]);
            g_error = why;
            return rc;
        }
    }
    return JH_OK;
}
JH_EXPORT int jh_step_commit(void* cv, int segments, const long long* ids, const int* lengths, int* released, int cap,
                             int* count) {
    Cache* c = static_cast<Cache*>(cv);
    std::vector<int> pairs;
    for (int i = 0; i < segments; ++i) {
        const int rc = c->commit(ids[i], lengths[i], &pairs);
        if (rc != JH_OK) return rc;
    }
    if (count) *count = (int)pairs.size() / 2;
    if (released) std::copy(pairs.begin(), pairs.begin() + std::min((int)pairs.size(), cap), released);
    return JH_OK;
}

// ---- the batch tables ---------------------------------------------------------------------------------------------------
JH_EXPORT void* jh_builder_new(int max_rows, int max_segments, int max_blocks, int groups, int page_size) {
    Builder* b = new Builder{max_rows, max_segments, max_blocks, groups, page_size, {}};
    b->rows.resize((size_t)std::max(1, groups) * max_segments);
    return b;
}
JH_EXPORT void jh_builder_delete(void* b) { delete static_cast<Builder*>(b); }

// Fills the pinned tables of one step. `small` holds, each `max_rows` long: token ids, positions, segment of the
// row, rows whose logits are wanted, then the cache row of every row per group; then, each `max_segments` long:
// first row, rows, positions held after the step, state slot of every segment. `tables` is [groups][max_segments]
// [max_blocks]. `wants` lists the wanted places of segment i at [want_at[i], want_at[i + 1]).
// info: rows, wanted rows, longest segment, most positions held, multi_segments (-1 if single rows come first), multi_rows.
JH_EXPORT int jh_builder_build(void* bv, void* cv, int segments, const long long* ids, const int* starts, const int* counts,
                               const int* tokens, const int* want_at, const int* wants, int vocab, int* small, int* tables,
                               int* info) {
    Builder* b = static_cast<Builder*>(bv);
    Cache* c = static_cast<Cache*>(cv);
    const int R = b->max_rows, S = b->max_segments, MB = b->max_blocks, G = b->groups, ps = b->page_size;
    if (segments == 0) return fail(JH_VALUE, "a step needs at least one segment");
    if (segments > S) return fail(JH_VALUE, "%d segments in one step, the engine was made for %d", segments, S);
    long long total = 0;
    for (int i = 0; i < segments; ++i) total += counts[i];
    if (total > R) return fail(JH_VALUE, "%lld rows in one step, the engine was made for %d", total, R);
    int *tok = small, *pos = small + R, *rseg = small + 2 * R, *lrows = small + 3 * R;
    int* seg_fields = small + (4 + G) * R;
    int *sstart = seg_fields, *slen = seg_fields + S, *skv = seg_fields + 2 * S, *sslot = seg_fields + 3 * S;
    int r = 0, n_want = 0, max_q = 0, max_kv = 0, multi_segments = 0, multi_rows = 0, t_at = 0;
    bool ordered = true;
    for (int si = 0; si < segments; ++si) {
        const long long id = ids[si];
        const int n = counts[si], start = starts[si];
        if (n < 1) return fail(JH_VALUE, "request #%lld: a segment needs at least one token", id);
        for (int sj = 0; sj < si; ++sj)
            if (ids[sj] == id) return fail(JH_VALUE, "request #%lld appears twice in one step", id);
        Request* rq = c->find(id);
        if (!rq) return fail(JH_KEY, "request #%lld is not open", id);
        for (int i = 0; i < n; ++i) {
            // a token id t < 0 says: row -t - 1 of the tokens that the step before this one sampled, which are still on
            // the device (`jllm_feed_tokens` puts it in place before the step runs); only a decoded token can be that
            const int t = tokens[t_at + i];
            if (t >= vocab || t < -S || (t < 0 && n != 1))
                return fail(JH_VALUE, "request #%lld: token id outside [0, %d)", id, vocab);
            tok[r + i] = t;
            pos[r + i] = start + i;
            rseg[r + i] = si;
        }
        t_at += n;
        sstart[si] = r;
        slen[si] = n;
        skv[si] = start + n;
        sslot[si] = rq->slot;
        for (int wi = want_at[si]; wi < want_at[si + 1]; ++wi) {
            const int w = wants[wi];
            if (w < 0 || w >= n) return fail(JH_VALUE, "request #%lld: wanted place %d is outside its %d tokens", id, w, n);
            lrows[n_want++] = r + w;
        }
        for (int g = 0; g < G; ++g) {
            const auto& table = rq->tables[g];
            const int nb = (int)table.size();
            if (nb > MB) return fail(JH_VALUE, "request #%lld holds %d pages, tables have %d columns", id, nb, MB);
            if ((long long)(start + n) > (long long)nb * ps)
                return fail(JH_VALUE, "request #%lld: positions up to %d have no pages (reserve first)", id, start + n);
            // the row of the host table: only what the request's table grew by since this row was last written for
            // it, if nothing else about the table changed (its epoch)
            Builder::Held& held = b->rows[(size_t)g * S + si];
            const int lo = (held.request == id && held.epoch == rq->epoch && held.entries <= nb) ? held.entries : 0;
            int* row = tables + ((size_t)g * S + si) * MB;
            std::copy(table.begin() + lo, table.end(), row + lo);
            held.request = id;
            held.epoch = rq->epoch;
            held.entries = nb;
            int* slots = small + (size_t)(4 + g) * R;
            for (int i = 0; i < n; ++i) {
                const int p = start + i;
                slots[r + i] = table[p / ps] * ps + p % ps;
            }
        }
        if (n > 1) {
            ordered = ordered && multi_segments == si;   // no single-row segment came before it
            multi_segments = si + 1;
            multi_rows = r + n;
        }
        r += n;
        max_q = std::max(max_q, n);
        max_kv = std::max(max_kv, start + n);
    }
    info[0] = r;
    info[1] = n_want;
    info[2] = max_q;
    info[3] = max_kv;
    info[4] = ordered ? multi_segments : -1;
    info[5] = multi_rows;
    return JH_OK;
}
