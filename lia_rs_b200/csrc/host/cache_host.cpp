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
// The request slots live here too (which are free, which are live, up to where each has pages), so that the
// scheduler's policy (scheduler_host.cpp) and the Python face `cache.CacheManager` see one state.
//
// Every function returns 0 or a count on success and a negative code on a refusal; `lia_host_error` gives the
// message of the last refusal on this thread.  Nothing here throws across the C boundary.
#include <stdio.h>
#include <string.h>

#include <new>

#include "cache_host.h"

#define LIA_HOST_EXPORT extern "C" __attribute__((visibility("default")))

using namespace lia_host;


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
    cache->live.assign((size_t)max_slots, 0);
    cache->length.assign((size_t)max_slots, 0);
    for (int slot = max_slots - 1; slot >= 0; --slot) cache->free_slots.push_back(slot);      // slot 0 first
    return cache;
}
LIA_HOST_EXPORT void lia_cache_destroy(void* cache) { delete static_cast<Cache*>(cache); }

LIA_HOST_EXPORT int lia_cache_available(void* handle, int group) { return static_cast<Cache*>(handle)->groups[(size_t)group].pool.available(); }

// ---- request slots ----
LIA_HOST_EXPORT int lia_cache_free_slots(void* handle) { return (int)static_cast<Cache*>(handle)->free_slots.size(); }
LIA_HOST_EXPORT int lia_cache_admit(void* handle) { return static_cast<Cache*>(handle)->admit(); }
LIA_HOST_EXPORT int lia_cache_is_live(void* handle, int slot) {
    Cache* cache = static_cast<Cache*>(handle);
    return !cache->bad_slot(slot) && cache->live[(size_t)slot];
}
LIA_HOST_EXPORT int lia_cache_length(void* handle, int slot) {
    Cache* cache = static_cast<Cache*>(handle);
    return cache->bad_slot(slot) ? refuse("slot outside the cache") : cache->length[(size_t)slot];
}
// For each of `n` slots: up to where it has pages, or -1 when it is not live (one call for a step's entries).
LIA_HOST_EXPORT int lia_cache_reserved(void* handle, const int* slots, int n, int* out) {
    Cache* cache = static_cast<Cache*>(handle);
    for (int i = 0; i < n; ++i)
        out[i] = (cache->bad_slot(slots[i]) || !cache->live[(size_t)slots[i]]) ? -1 : cache->length[(size_t)slots[i]];
    return 0;
}
// The free slots into `out` (room for max_slots), in the order of the list; returns how many.
LIA_HOST_EXPORT int lia_cache_free_slot_list(void* handle, int* out) {
    Cache* cache = static_cast<Cache*>(handle);
    for (size_t i = 0; i < cache->free_slots.size(); ++i) out[i] = cache->free_slots[i];
    return (int)cache->free_slots.size();
}

// Free pages that ensure(slot, start, end) would need in the tightest group, counting what it would first give back.
LIA_HOST_EXPORT int lia_cache_pages_for(void* handle, int slot, int start, int end) {
    return static_cast<Cache*>(handle)->pages_for(slot, start, end);
}

// Pages for positions [start, end) of the live slot `slot` in every group, all or nothing: 1 done, 0 some group has too
// few free pages (nothing was changed), negative a refusal.
LIA_HOST_EXPORT int lia_cache_ensure(void* handle, int slot, int start, int end, int max_context) {
    return static_cast<Cache*>(handle)->ensure(slot, start, end, max_context);
}

// The slot's pages are given back and the slot is free again.
LIA_HOST_EXPORT int lia_cache_release_slot(void* handle, int slot) { return static_cast<Cache*>(handle)->release(slot); }

// The table of `slot` in `group` (page per logical block, -1: none) into `out` (up to `capacity` entries); returns
// its length.
LIA_HOST_EXPORT int lia_cache_table(void* handle, int group, int slot, int* out, int capacity) {
    Cache* cache = static_cast<Cache*>(handle);
    if (cache->bad_slot(slot)) return refuse("slot outside the cache");
    const std::vector<int>& table = cache->groups[(size_t)group].tables[(size_t)slot];
    for (size_t b = 0; b < table.size() && (int)b < capacity; ++b) out[b] = table[b];
    return (int)table.size();
}
LIA_HOST_EXPORT int lia_cache_first_block(void* handle, int group, int slot) {
    Cache* cache = static_cast<Cache*>(handle);
    if (cache->bad_slot(slot)) return refuse("slot outside the cache");
    return cache->groups[(size_t)group].first_block[(size_t)slot];
}
// Pages that the table of `slot` holds in `group`.
LIA_HOST_EXPORT int lia_cache_held(void* handle, int group, int slot) {
    Cache* cache = static_cast<Cache*>(handle);
    if (cache->bad_slot(slot)) return refuse("slot outside the cache");
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
        if (cache->bad_slot(slot)) return refuse("slot outside the cache");
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
