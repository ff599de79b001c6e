// Host bookkeeping of the paged cache, native: pools of pages (a free list and a user count per page) and, per
// group of layers, the block table of every request slot.  No CUDA in this file; the Python classes
// `cache.PagePool` and `cache.CacheGroup` are its faces and own the tensors.
//
// The reference keeps the same state in its page cache (src/inference/page_cache.rs:12-16, 184-206, 240-245:
// users per page, underflow refused, allocation all or nothing) and uploads the block table before a step
// (src/inference/paging.rs:224-237).  Here a group writes every change of a table entry straight into the
// pinned host copy of the table (`host_table`, given at creation) and remembers, per slot, the range of blocks
// that changed since the last `lia_cache_take_dirty`, so that only those go to the device.
//
// Every function returns 0 or a count on success and a negative code on a refusal; `lia_host_error` gives the
// message of the last refusal on this thread.  Nothing here throws across the C boundary.
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <new>
#include <string>
#include <vector>

#define LIA_HOST_EXPORT extern "C" __attribute__((visibility("default")))

namespace {
thread_local std::string last_error;

int refuse(const std::string& message) {
    last_error = message;
    return -1;
}

struct Pool {
    int num_pages = 0;
    std::vector<int> free_list;          // back() is handed out next: a page just given back is used again first
    std::vector<int> users;

    explicit Pool(int n) : num_pages(n), users((size_t)n, 0) {
        free_list.reserve((size_t)n);
        for (int page = n - 1; page >= 0; --page) free_list.push_back(page);     // page 0 first
    }
    int available() const { return (int)free_list.size(); }
    int allocate() {
        if (free_list.empty()) return refuse("page pool exhausted");
        const int page = free_list.back();
        if (users[(size_t)page] != 0) return refuse("page " + std::to_string(page) + " on the free list is held");
        free_list.pop_back();
        users[(size_t)page] = 1;
        return page;
    }
    int release(int page) {
        if (page < 0 || page >= num_pages) return refuse("page " + std::to_string(page) + " is outside the pool");
        if (users[(size_t)page] <= 0) return refuse("page " + std::to_string(page) + " freed twice");
        if (--users[(size_t)page] == 0) free_list.push_back(page);
        return 0;
    }
    // Every page is on the free list once or held by exactly the given holders (`held`: the pages the block tables hold).
    int check(const std::vector<int>& held) const {
        std::vector<int> on_free((size_t)num_pages, 0), holders((size_t)num_pages, 0);
        for (int page : free_list) {
            if (page < 0 || page >= num_pages) return refuse("the free list names page " + std::to_string(page));
            if (++on_free[(size_t)page] > 1) return refuse("a page is on the free list twice");
        }
        for (int page : held) {
            if (page < 0 || page >= num_pages) return refuse("a block table names page " + std::to_string(page));
            ++holders[(size_t)page];
        }
        for (int page = 0; page < num_pages; ++page) {
            if (users[(size_t)page] != holders[(size_t)page])
                return refuse("page " + std::to_string(page) + ": " + std::to_string(users[(size_t)page]) + " users recorded, " +
                              std::to_string(holders[(size_t)page]) + " holders found");
            if ((holders[(size_t)page] == 0) != (on_free[(size_t)page] == 1))
                return refuse("page " + std::to_string(page) + " is lost or both held and free");
        }
        return 0;
    }
};

struct Plan {
    std::vector<int> allocate, give_back;
    int keep_from = 0;
};

struct Group {
    Pool pool;
    int page_size, window, max_slots, max_blocks;      // window < 0: all keys
    int32_t* host_table;                               // [max_slots, max_blocks], -1: no page
    std::vector<std::vector<int>> tables;              // per slot: page of each logical block, or -1
    std::vector<int> first_block;                      // blocks before this were given back
    std::vector<int> dirty_lo, dirty_hi;               // per slot: the range of blocks to copy (lo < 0: none)
    std::vector<int> dirty_slots;                      // slots with a range, in the order they became dirty

    Group(int pages, int page_size_, int window_, int slots, int blocks, int32_t* table)
        : pool(pages), page_size(page_size_), window(window_), max_slots(slots), max_blocks(blocks), host_table(table),
          tables((size_t)slots), first_block((size_t)slots, 0), dirty_lo((size_t)slots, -1), dirty_hi((size_t)slots, 0) {}

    void mark(int slot, int lo, int hi) {
        if (dirty_lo[(size_t)slot] < 0) {
            dirty_lo[(size_t)slot] = lo;
            dirty_hi[(size_t)slot] = hi;
            dirty_slots.push_back(slot);
        } else {
            dirty_lo[(size_t)slot] = std::min(dirty_lo[(size_t)slot], lo);
            dirty_hi[(size_t)slot] = std::max(dirty_hi[(size_t)slot], hi);
        }
    }
    // The blocks of a slot's table from first_block on are all present (blocks are only ever given back from the
    // front, and allocated without gaps), so only the table's ends are looked at: a decode step costs the same
    // whatever the context length.
    void needed(int slot, int start, int end, Plan* plan) const {
        const std::vector<int>& table = tables[(size_t)slot];
        const int n = (int)table.size(), first = first_block[(size_t)slot];
        int keep_from = 0;
        if (window >= 0) keep_from = std::max(0, start - window + 1) / page_size;
        plan->allocate.clear();
        plan->give_back.clear();
        plan->keep_from = keep_from;
        for (int b = first; b < std::min(keep_from, n); ++b)
            if (table[(size_t)b] >= 0) plan->give_back.push_back(b);
        const int last = (end - 1) / page_size;
        for (int b = keep_from; b < std::min(first, last + 1); ++b) plan->allocate.push_back(b);       // given back earlier, wanted again
        for (int b = std::max(keep_from, n); b <= last; ++b) plan->allocate.push_back(b);              // beyond the table's end
    }
    // The same by looking at every block (what the invariant check compares `needed` with).
    void needed_by_scan(int slot, int start, int end, Plan* plan) const {
        const std::vector<int>& table = tables[(size_t)slot];
        const int n = (int)table.size();
        int keep_from = 0;
        if (window >= 0) keep_from = std::max(0, start - window + 1) / page_size;
        plan->allocate.clear();
        plan->give_back.clear();
        plan->keep_from = keep_from;
        for (int b = first_block[(size_t)slot]; b < std::min(keep_from, n); ++b)
            if (table[(size_t)b] >= 0) plan->give_back.push_back(b);
        const int last = (end - 1) / page_size;
        for (int b = keep_from; b <= last; ++b)
            if (b >= n || table[(size_t)b] < 0) plan->allocate.push_back(b);
    }
    int apply(int slot, const Plan& plan) {
        std::vector<int>& table = tables[(size_t)slot];
        int32_t* row = host_table + (size_t)slot * max_blocks;
        for (int b : plan.give_back) {
            if (pool.release(table[(size_t)b]) < 0) return -1;
            table[(size_t)b] = -1;
            row[b] = -1;
            mark(slot, b, b + 1);
        }
        first_block[(size_t)slot] = std::max(first_block[(size_t)slot], std::min(plan.keep_from, (int)table.size()));
        for (int b : plan.allocate) {
            if (b >= max_blocks) return refuse("block " + std::to_string(b) + " is beyond the table's " + std::to_string(max_blocks));
            while ((int)table.size() <= b) table.push_back(-1);
            const int page = pool.allocate();
            if (page < 0) return -1;
            table[(size_t)b] = page;
            row[b] = page;
            mark(slot, b, b + 1);
        }
        return 0;
    }
    int release_slot(int slot) {
        std::vector<int>& table = tables[(size_t)slot];
        for (int page : table)
            if (page >= 0 && pool.release(page) < 0) return -1;
        if (!table.empty()) {
            int32_t* row = host_table + (size_t)slot * max_blocks;
            for (size_t b = 0; b < table.size(); ++b) row[b] = -1;
            mark(slot, 0, (int)table.size());
        }
        table.clear();
        first_block[(size_t)slot] = 0;
        return 0;
    }
};

struct Cache {
    std::vector<Group> groups;
    int max_slots = 0;
    std::vector<Plan> plans;             // scratch of ensure
};

bool bad_slot(const Cache* cache, int slot) { return slot < 0 || slot >= cache->max_slots; }
}  // namespace

LIA_HOST_EXPORT const char* lia_host_error() { return last_error.c_str(); }

// ---- a pool on its own (the face `cache.PagePool`) ----
LIA_HOST_EXPORT void* lia_pool_create(int num_pages) {
    if (num_pages <= 0) { refuse("empty page pool"); return nullptr; }
    return new (std::nothrow) Pool(num_pages);
}
LIA_HOST_EXPORT void lia_pool_destroy(void* pool) { delete static_cast<Pool*>(pool); }
LIA_HOST_EXPORT int lia_pool_available(void* pool) { return static_cast<Pool*>(pool)->available(); }
LIA_HOST_EXPORT int lia_pool_allocate(void* pool) { return static_cast<Pool*>(pool)->allocate(); }
LIA_HOST_EXPORT int lia_pool_release(void* pool, int page) { return static_cast<Pool*>(pool)->release(page); }
LIA_HOST_EXPORT int lia_pool_users(void* pool, int page) {
    Pool* p = static_cast<Pool*>(pool);
    return page >= 0 && page < p->num_pages ? p->users[(size_t)page] : refuse("page outside the pool");
}
LIA_HOST_EXPORT int lia_pool_check(void* pool, const int* held, int n_held) {
    return static_cast<Pool*>(pool)->check(std::vector<int>(held, held + n_held));
}

// ---- the groups of a cache manager ----
// `windows[g]` < 0: the group keeps all keys.  `host_tables[g]`: int32 [max_slots, max_blocks], owned by the caller,
// filled with -1; the cache writes the entries it changes.
LIA_HOST_EXPORT void* lia_cache_create(int n_groups, const int* num_pages, const int* page_sizes, const int* windows,
                                       int max_slots, int max_blocks, int32_t* const* host_tables) {
    if (n_groups < 0 || max_slots <= 0 || max_blocks <= 0) { refuse("sizes of the cache must be positive"); return nullptr; }
    Cache* cache = new (std::nothrow) Cache();
    if (!cache) return nullptr;
    cache->max_slots = max_slots;
    for (int g = 0; g < n_groups; ++g) {
        if (num_pages[g] <= 0 || page_sizes[g] <= 0 || !host_tables[g]) {
            delete cache;
            refuse("empty page pool");
            return nullptr;
        }
        cache->groups.emplace_back(num_pages[g], page_sizes[g], windows[g], max_slots, max_blocks, host_tables[g]);
    }
    cache->plans.resize((size_t)n_groups);
    return cache;
}
LIA_HOST_EXPORT void lia_cache_destroy(void* cache) { delete static_cast<Cache*>(cache); }

LIA_HOST_EXPORT int lia_cache_available(void* handle, int group) { return static_cast<Cache*>(handle)->groups[(size_t)group].pool.available(); }

// Free pages that ensure(slot, start, end) would need in the tightest group, counting what it would first give back.
LIA_HOST_EXPORT int lia_cache_pages_for(void* handle, int slot, int start, int end) {
    Cache* cache = static_cast<Cache*>(handle);
    if (bad_slot(cache, slot)) return refuse("slot outside the cache");
    int worst = 0;
    Plan plan;
    for (Group& group : cache->groups) {
        if (group.window < 0 && (end - 1) / group.page_size < (int)group.tables[(size_t)slot].size()) continue;
        group.needed(slot, start, end, &plan);
        worst = std::max(worst, (int)plan.allocate.size() - (int)plan.give_back.size());
    }
    return worst;
}

// Pages for positions [start, end) of `slot` in every group, all or nothing: 1 done, 0 some group has too few free
// pages (nothing was changed), negative a refusal.
LIA_HOST_EXPORT int lia_cache_ensure(void* handle, int slot, int start, int end) {
    Cache* cache = static_cast<Cache*>(handle);
    if (bad_slot(cache, slot)) return refuse("slot outside the cache");
    bool present = true;
    for (const Group& group : cache->groups)
        present = present && group.window < 0 && (end - 1) / group.page_size < (int)group.tables[(size_t)slot].size();
    if (present) return 1;                               // every position already has its page (most decode steps)
    for (size_t g = 0; g < cache->groups.size(); ++g) {
        Group& group = cache->groups[g];
        group.needed(slot, start, end, &cache->plans[g]);
        if ((int)cache->plans[g].allocate.size() - (int)cache->plans[g].give_back.size() > group.pool.available()) return 0;
    }
    for (size_t g = 0; g < cache->groups.size(); ++g)
        if (cache->groups[g].apply(slot, cache->plans[g]) < 0) return -1;
    return 1;
}

LIA_HOST_EXPORT int lia_cache_release_slot(void* handle, int slot) {
    Cache* cache = static_cast<Cache*>(handle);
    if (bad_slot(cache, slot)) return refuse("slot outside the cache");
    for (Group& group : cache->groups)
        if (group.release_slot(slot) < 0) return -1;
    return 0;
}

// The table of `slot` in `group` (page per logical block, -1: none) into `out` (up to `capacity` entries); returns
// its length.
LIA_HOST_EXPORT int lia_cache_table(void* handle, int group, int slot, int* out, int capacity) {
    Cache* cache = static_cast<Cache*>(handle);
    if (bad_slot(cache, slot)) return refuse("slot outside the cache");
    const std::vector<int>& table = cache->groups[(size_t)group].tables[(size_t)slot];
    for (size_t b = 0; b < table.size() && (int)b < capacity; ++b) out[b] = table[b];
    return (int)table.size();
}
LIA_HOST_EXPORT int lia_cache_first_block(void* handle, int group, int slot) {
    Cache* cache = static_cast<Cache*>(handle);
    if (bad_slot(cache, slot)) return refuse("slot outside the cache");
    return cache->groups[(size_t)group].first_block[(size_t)slot];
}
// Pages that the table of `slot` holds in `group`.
LIA_HOST_EXPORT int lia_cache_held(void* handle, int group, int slot) {
    Cache* cache = static_cast<Cache*>(handle);
    if (bad_slot(cache, slot)) return refuse("slot outside the cache");
    int held = 0;
    for (int page : cache->groups[(size_t)group].tables[(size_t)slot]) held += page >= 0;
    return held;
}

// The ranges of blocks that changed since the last call, as (slot, lo, hi) triples into `out` (room for `capacity`
// triples: max_slots is enough); returns how many, and forgets them.
LIA_HOST_EXPORT int lia_cache_take_dirty(void* handle, int group, int* out, int capacity) {
    Group& g = static_cast<Cache*>(handle)->groups[(size_t)group];
    int n = 0;
    for (int slot : g.dirty_slots) {
        if (n < capacity) {
            out[3 * n] = slot;
            out[3 * n + 1] = g.dirty_lo[(size_t)slot];
            out[3 * n + 2] = g.dirty_hi[(size_t)slot];
            ++n;
        }
        g.dirty_lo[(size_t)slot] = -1;
        g.dirty_hi[(size_t)slot] = 0;
    }
    g.dirty_slots.clear();
    return n;
}

// The invariants of one group: no page lost, none held twice, none both free and held; for the live slots the
// table's shape that `needed` relies on, and `needed` against a scan of the table at the slot's length.
LIA_HOST_EXPORT int lia_cache_check(void* handle, int group, const int* live_slots, const int* lengths, int n_live, int max_context) {
    Cache* cache = static_cast<Cache*>(handle);
    Group& g = cache->groups[(size_t)group];
    std::vector<int> held;
    for (const std::vector<int>& table : g.tables)
        for (int page : table)
            if (page >= 0) held.push_back(page);
    std::vector<int> sorted(held);
    std::sort(sorted.begin(), sorted.end());
    if (std::adjacent_find(sorted.begin(), sorted.end()) != sorted.end())
        return refuse("group " + std::to_string(group) + ": a page is held twice");
    if (g.pool.check(held) < 0) return -1;
    Plan fast, scan;
    for (int i = 0; i < n_live; ++i) {
        const int slot = live_slots[i];
        if (bad_slot(cache, slot)) return refuse("slot outside the cache");
        const std::vector<int>& table = g.tables[(size_t)slot];
        const int first = g.first_block[(size_t)slot];
        for (int b = 0; b < (int)table.size(); ++b)
            if ((b < first) != (table[(size_t)b] < 0))
                return refuse("group " + std::to_string(group) + ", slot " + std::to_string(slot) + ": the block table has a gap");
        if (lengths[i] < max_context) {
            g.needed(slot, lengths[i], lengths[i] + 1, &fast);
            g.needed_by_scan(slot, lengths[i], lengths[i] + 1, &scan);
            if (fast.allocate != scan.allocate || fast.give_back != scan.give_back || fast.keep_from != scan.keep_from)
                return refuse("group " + std::to_string(group) + ", slot " + std::to_string(slot) +
                              ": pages_needed disagrees with a scan of the table");
        }
    }
    return 0;
}
