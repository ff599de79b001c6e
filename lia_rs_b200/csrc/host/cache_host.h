// The paged cache's host bookkeeping as C++ types, shared by its C interface (cache_host.cpp) and by the scheduler's
// policy (scheduler_host.cpp).  See cache_host.cpp for what they are.
#pragma once
#include <stdint.h>

#include <algorithm>
#include <string>
#include <vector>

namespace lia_host {
inline thread_local std::string last_error;

inline int refuse(const std::string& message) {
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
    // request slots: which are free (back() is handed out next), which are live, and up to where each has pages
    std::vector<int> free_slots;
    std::vector<char> live;
    std::vector<int> length;             // positions [0, length) of a live slot have been ensured

    bool bad_slot(int slot) const { return slot < 0 || slot >= max_slots; }
    int available() const {              // free pages of the tightest group
        int fewest = 1 << 30;
        for (const Group& group : groups) fewest = std::min(fewest, group.pool.available());
        return fewest;
    }
    int admit() {
        if (free_slots.empty()) return refuse("no free request slot");
        const int slot = free_slots.back();
        free_slots.pop_back();
        live[(size_t)slot] = 1;
        length[(size_t)slot] = 0;
        return slot;
    }
    // Free pages that ensure(slot, start, end) would need in the tightest group, counting what it would first give back.
    int pages_for(int slot, int start, int end) {
        if (bad_slot(slot)) return refuse("slot outside the cache");
        int worst = 0;
        Plan plan;
        for (Group& group : groups) {
            if (group.window < 0 && (end - 1) / group.page_size < (int)group.tables[(size_t)slot].size()) continue;
            group.needed(slot, start, end, &plan);
            worst = std::max(worst, (int)plan.allocate.size() - (int)plan.give_back.size());
        }
        return worst;
    }
    // Pages for positions [start, end) of `slot` in every group, all or nothing: 1 done, 0 some group has too few free
    // pages (nothing was changed), negative a refusal.
    int ensure(int slot, int start, int end, int max_context) {
        if (bad_slot(slot) || !live[(size_t)slot]) return refuse("slot " + std::to_string(slot) + " is not live");
        if (!(0 <= start && start < end) || end > max_context)
            return refuse("positions [" + std::to_string(start) + ", " + std::to_string(end) + ") are outside the context of " + std::to_string(max_context));
        bool present = true;
        for (const Group& group : groups)
            present = present && group.window < 0 && (end - 1) / group.page_size < (int)group.tables[(size_t)slot].size();
        if (!present) {                                  // (most decode steps find every position's page there)
            for (size_t g = 0; g < groups.size(); ++g) {
                groups[g].needed(slot, start, end, &plans[g]);
                if ((int)plans[g].allocate.size() - (int)plans[g].give_back.size() > groups[g].pool.available()) return 0;
            }
            for (size_t g = 0; g < groups.size(); ++g)
                if (groups[g].apply(slot, plans[g]) < 0) return -1;
        }
        length[(size_t)slot] = std::max(length[(size_t)slot], end);
        return 1;
    }
    int release(int slot) {
        if (bad_slot(slot) || !live[(size_t)slot]) return refuse("slot " + std::to_string(slot) + " released twice or never admitted");
        for (Group& group : groups)
            if (group.release_slot(slot) < 0) return -1;
        live[(size_t)slot] = 0;
        length[(size_t)slot] = 0;
        free_slots.push_back(slot);
        return 0;
    }
    int held(int slot) const {           // pages of the group that holds most for this slot
        int most = 0;
        for (const Group& group : groups) {
            int held = 0;
            for (int page : group.tables[(size_t)slot]) held += page >= 0;
            most = std::max(most, held);
        }
        return most;
    }
};
}  // namespace lia_host
