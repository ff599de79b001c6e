// The scheduler's policy, native: which requests get a slot, who gives way when pages run out, and which tokens of
// which request a step runs.  No CUDA in this file; it works on the cache's native bookkeeping (cache_host.h) and
// knows a request only by its counts: tokens held, tokens computed, tokens generated, its limit, its slot.  The
// Python class `engine.Scheduler` is its face: it owns the token lists, the samplers and the clock, asks this
// core what to do, runs the step and reports what was accepted.
//
// The policy is the reference's continuous-batching loop (src/server/paged.rs:64-99,
// src/server/paged/{request,schedule,preempt}.rs):
//   admission   first come, first served, paused requests before queued ones; a request gets a slot when one is
//               free and the page of its first token can be had, a paused one only when its whole prefix fits
//               again (request.rs:6-24,85-88; preempt.rs:5-21,38-42); otherwise it stays at the head and
//               admission stops
//   capacity    before each step, while more live requests need a new page than pages are free, one is preempted:
//               the one that has already produced a token, then holds most pages, then sits in the highest slot;
//               its pages go back, it keeps its tokens and is computed again from position 0 when it is resumed;
//               a single request that cannot fit is an error (preempt.rs:61-113)
//   the step    single decoded tokens first, the rest of the budget to prompt portions in slot order; or, with
//               even_split, max(1, budget / live) tokens for every live request (schedule.rs:11,28-50); a portion
//               is shortened at the first page that cannot be had (schedule.rs:30-36)
//
// Every function returns 0 or a count on success and a negative code on a refusal (`lia_host_error` has the message).
#include <deque>
#include <new>

#include "cache_host.h"

#define LIA_HOST_EXPORT extern "C" __attribute__((visibility("default")))

using namespace lia_host;

namespace {
struct Request {
    int tokens = 0;          // prompt and accepted tokens that are fed back
    int computed = 0;        // of them, those whose keys and values are in the cache
    int generated = 0;
    int max_tokens = 0;
    int slot = -1;
    int preemptions = 0;
    bool done = false;
};

struct Scheduler {
    Cache* cache = nullptr;
    int budget = 0, max_context = 0, page_size = 1;
    bool even_split = false;
    std::vector<Request> requests;
    std::deque<int> queue, paused;
    std::vector<int> active;         // request by slot, or -1

    int live(std::vector<int>* out) const {
        out->clear();
        for (int request : active)
            if (request >= 0) out->push_back(request);
        return (int)out->size();
    }
    // A slot and the page of the first uncomputed token, or nothing.
    int attach(int request) {
        if (cache->free_slots.empty()) return 0;
        const int slot = cache->admit();
        if (slot < 0) return -1;
        const int had = cache->ensure(slot, 0, 1, max_context);
        if (had <= 0) {
            if (cache->release(slot) < 0) return -1;
            return had;
        }
        requests[(size_t)request].slot = slot;
        requests[(size_t)request].computed = 0;
        active[(size_t)slot] = request;
        return 1;
    }
    // How many of the request's next tokens (at most `allowance`) have pages: the portion is cut at the first page
    // that cannot be had.
    int portion(const Request& r, int allowance) {
        const int start = r.computed;
        int want = std::min(allowance, r.tokens - start);
        while (want > 0) {
            const int had = cache->ensure(r.slot, start, start + want, max_context);
            if (had < 0) return -1;
            if (had) break;
            const int boundary = ((start + want - 1) / page_size) * page_size;      // the end of the last page that may still be had
            want = boundary > start ? boundary - start : 0;
        }
        return want;
    }
};

enum Event { ATTACHED_FROM_QUEUE = 1, PREEMPTED = 2, ATTACHED_FROM_PAUSED = 3 };

Scheduler* of(void* handle) { return static_cast<Scheduler*>(handle); }
bool bad_request(const Scheduler* s, int request) { return request < 0 || request >= (int)s->requests.size(); }
}  // namespace

LIA_HOST_EXPORT void* lia_sched_create(void* cache, int budget, int even_split, int max_context, int page_size) {
    if (!cache || budget <= 0 || max_context <= 0 || page_size <= 0) { refuse("the scheduler's sizes must be positive"); return nullptr; }
    Scheduler* s = new (std::nothrow) Scheduler();
    if (!s) return nullptr;
    s->cache = static_cast<Cache*>(cache);
    s->budget = budget;
    s->even_split = even_split != 0;
    s->max_context = max_context;
    s->page_size = page_size;
    s->active.assign((size_t)s->cache->max_slots, -1);
    return s;
}
LIA_HOST_EXPORT void lia_sched_destroy(void* handle) { delete of(handle); }

// A request of `tokens` prompt tokens that may generate `max_tokens`, queued; returns its number.
LIA_HOST_EXPORT int lia_sched_add(void* handle, int tokens, int max_tokens) {
    Scheduler* s = of(handle);
    if (tokens <= 0 || max_tokens <= 0) return refuse("a request needs a prompt and a positive token limit");
    Request r;
    r.tokens = tokens;
    r.max_tokens = max_tokens;
    s->requests.push_back(r);
    s->queue.push_back((int)s->requests.size() - 1);
    return (int)s->requests.size() - 1;
}

// Admission, then room for the step: what happened goes into `events` as (kind, request, slot) triples (room for
// `capacity` of them; the slot of a preempted request is the one it lost).  Returns their number.
LIA_HOST_EXPORT int lia_sched_prepare(void* handle, int* events, int capacity) {
    Scheduler* s = of(handle);
    int n = 0;
    auto note = [&](int kind, int request, int slot) {
        if (n < capacity) {
            events[3 * n] = kind;
            events[3 * n + 1] = request;
            events[3 * n + 2] = slot;
        }
        ++n;
    };
    // ---- admission ----
    while (!s->cache->free_slots.empty()) {
        if (!s->paused.empty()) {
            const int request = s->paused.front();
            // a paused request is not taken back before its whole prefix fits again
            const int needed = (s->requests[(size_t)request].tokens + s->page_size - 1) / s->page_size;
            if (needed > s->cache->available()) break;
            const int got = s->attach(request);
            if (got < 0) return -1;
            if (!got) break;
            s->paused.pop_front();
            note(ATTACHED_FROM_PAUSED, request, s->requests[(size_t)request].slot);
            continue;
        }
        if (s->queue.empty()) break;
        const int request = s->queue.front();
        const int got = s->attach(request);
        if (got < 0) return -1;
        if (!got) break;
        s->queue.pop_front();
        note(ATTACHED_FROM_QUEUE, request, s->requests[(size_t)request].slot);
    }
    // ---- pages run out ----
    std::vector<int> live;
    for (;;) {
        s->live(&live);
        int needed = 0;
        for (int request : live) {
            const Request& r = s->requests[(size_t)request];
            if (r.done) continue;
            const int pages = s->cache->pages_for(r.slot, r.computed, r.computed + 1);
            if (pages < 0) return -1;
            needed += pages > 0;
        }
        if (needed <= s->cache->available()) break;
        if (live.size() <= 1) { refuse("one request exceeded its physical KV capacity"); return -2; }
        int victim = -1, victim_held = 0;
        for (int request : live) {
            const Request& r = s->requests[(size_t)request];
            const int held = s->cache->held(r.slot);
            bool better = victim < 0;
            if (!better) {
                const Request& v = s->requests[(size_t)victim];
                if ((r.generated > 0) != (v.generated > 0)) better = r.generated > 0;
                else if (held != victim_held) better = held > victim_held;
                else better = r.slot > v.slot;
            }
            if (better) { victim = request; victim_held = held; }
        }
        Request& v = s->requests[(size_t)victim];
        const int slot = v.slot;
        if (s->cache->release(slot) < 0) return -1;
        s->active[(size_t)slot] = -1;
        v.slot = -1;
        v.computed = 0;
        ++v.preemptions;
        s->paused.push_back(victim);
        note(PREEMPTED, victim, slot);
    }
    return n;
}

// The step: (request, start, count, is this the request's last uncomputed token) quadruples into `out` (room for
// `capacity`), their pages reserved.  Returns their number; 0 with live requests that are not done means that
// nothing can be run.
LIA_HOST_EXPORT int lia_sched_plan(void* handle, int* out, int capacity) {
    Scheduler* s = of(handle);
    std::vector<int> live;
    if (s->live(&live) == 0) return 0;
    int n = 0;
    auto take = [&](int request, int count) {
        const Request& r = s->requests[(size_t)request];
        if (n < capacity) {
            out[4 * n] = request;
            out[4 * n + 1] = r.computed;
            out[4 * n + 2] = count;
            out[4 * n + 3] = r.computed + count == r.tokens;
        }
        ++n;
    };
    if (s->even_split) {
        const int allowance = std::max(1, s->budget / (int)live.size());
        for (int request : live) {
            const int count = s->portion(s->requests[(size_t)request], allowance);
            if (count < 0) return -1;
            if (count) take(request, count);
        }
        return n;
    }
    int budget = s->budget;
    for (int request : live) {                           // single decoded tokens first
        const Request& r = s->requests[(size_t)request];
        if (r.tokens - r.computed != 1) continue;
        if (budget <= 0) break;
        const int count = s->portion(r, 1);
        if (count < 0) return -1;
        if (count) { take(request, 1); --budget; }
    }
    for (int request : live) {                           // then portions of prompts, in slot order
        const Request& r = s->requests[(size_t)request];
        if (r.tokens - r.computed <= 1) continue;
        if (budget <= 0) break;
        const int count = s->portion(r, budget);
        if (count < 0) return -1;
        if (count) { take(request, count); budget -= count; }
    }
    return n;
}

// `count` more tokens of the request are in the cache.
LIA_HOST_EXPORT int lia_sched_advance(void* handle, int request, int count) {
    Scheduler* s = of(handle);
    if (bad_request(s, request)) return refuse("no such request");
    Request& r = s->requests[(size_t)request];
    // (one more than it holds: in pipelined decoding the token of the step before is fed on the device and accepted
    // on the host only after the next step has been launched)
    if (count < 0 || r.computed + count > r.tokens + 1) return refuse("more tokens computed than the request holds");
    r.computed += count;
    return 0;
}

// A token was accepted: the request is done (`done`) or the token is fed back.
LIA_HOST_EXPORT int lia_sched_accept(void* handle, int request, int done) {
    Scheduler* s = of(handle);
    if (bad_request(s, request)) return refuse("no such request");
    Request& r = s->requests[(size_t)request];
    ++r.generated;
    r.done = done != 0;
    if (!r.done) ++r.tokens;
    return 0;
}

// What the finished requests hold is freed; their numbers go into `out` (room for a request per slot), in slot
// order.  Returns how many.
LIA_HOST_EXPORT int lia_sched_retire(void* handle, int* out) {
    Scheduler* s = of(handle);
    int n = 0;
    for (size_t slot = 0; slot < s->active.size(); ++slot) {
        const int request = s->active[slot];
        if (request < 0 || !s->requests[(size_t)request].done) continue;
        if (s->cache->release((int)slot) < 0) return -1;
        s->active[slot] = -1;
        s->requests[(size_t)request].slot = -1;
        out[n++] = request;
    }
    return n;
}

// Whether the step after a pending decode step of `requests` (in slot order) is known before that step's tokens
// are: nothing waits, every live request is one of them and decodes on whatever token it gets (short of an end of
// sequence), and the pages suffice.
LIA_HOST_EXPORT int lia_sched_can_continue(void* handle, const int* requests, int n) {
    Scheduler* s = of(handle);
    std::vector<int> live;
    s->live(&live);
    if (!s->queue.empty() || !s->paused.empty() || (int)live.size() != n || n > s->budget) return 0;
    int needed = 0;
    for (int i = 0; i < n; ++i) {
        if (live[(size_t)i] != requests[i]) return 0;
        const Request& r = s->requests[(size_t)requests[i]];
        if (r.done || r.tokens != r.computed) return 0;
        if (r.generated + 1 >= r.max_tokens) return 0;   // the pending token is its last
        const int pages = s->cache->pages_for(r.slot, r.computed, r.computed + 1);
        if (pages < 0) return -1;
        needed += pages > 0;
    }
    return needed <= s->cache->available();
}

// The page of each of these requests' next position, for a step whose tokens are fed on the device.
LIA_HOST_EXPORT int lia_sched_reserve_next(void* handle, const int* requests, int n) {
    Scheduler* s = of(handle);
    for (int i = 0; i < n; ++i) {
        if (bad_request(s, requests[i])) return refuse("no such request");
        const Request& r = s->requests[(size_t)requests[i]];
        const int had = s->cache->ensure(r.slot, r.computed, r.computed + 1, s->max_context);
        if (had < 0) return -1;
        if (!had) return refuse("a page that was counted free could not be had");
    }
    return 0;
}

// (slot, computed, tokens, generated, done, preemptions) of a request.
LIA_HOST_EXPORT int lia_sched_request(void* handle, int request, int* out) {
    Scheduler* s = of(handle);
    if (bad_request(s, request)) return refuse("no such request");
    const Request& r = s->requests[(size_t)request];
    out[0] = r.slot; out[1] = r.computed; out[2] = r.tokens; out[3] = r.generated; out[4] = r.done; out[5] = r.preemptions;
    return 0;
}

// (queued, paused, live) requests.
LIA_HOST_EXPORT int lia_sched_counts(void* handle, int* out) {
    Scheduler* s = of(handle);
    std::vector<int> live;
    out[0] = (int)s->queue.size();
    out[1] = (int)s->paused.size();
    out[2] = s->live(&live);
    return 0;
}
