"""The cache manager: keys and values in pages with a block table per request, one group of
pages per kind of need, and slots of fixed-size per-request state.

* A *slot* is the place of a live request (0 .. max_slots-1): its row in every block table and in
  every state tensor.
* A *group* collects the caches (one per attention layer that writes one) whose need is the same
  (kv heads, head size, all keys or a window).  A group has one pool of pages and one block table;
  each of its caches has its own K and V tensors [pages, page_size, kv_heads, head_dim] indexed by
  the same page numbers.  Different groups have pages of their own.
* `ensure(slot, start, end)` makes the pages for positions [start, end) present in every group,
  all or nothing (src/inference/page_cache.rs:184-206).  In a window group the pages that lie
  wholly before `start - window + 1` are given back first: no later token can see them.
* `release(slot)` gives everything back (request finished, aborted or preempted:
  src/server/paged/schedule.rs:134, preempt.rs:73,108).
* Block tables live on the host and on the device; `flush()` copies the rows that changed.  The copies are
  asynchronous and read a snapshot of those rows taken at `flush()` (a small ring of pinned staging buffers,
  each guarded by an event), never the live table: the host may go on changing the table (reserve pages for
  the step after, release a request that ended) while the copies of an earlier step are still queued.  The
  reference uploads the whole table before each step and waits (src/inference/paging.rs:224-237).
  A table entry of -1 means "no page" (never allocated, or passed by the window).

The manager is pure bookkeeping plus tensors; it runs on the CPU device too, which is how its
tests exercise it without a GPU.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .pages import PageError, PagePool


@dataclass
class KVView:
    """What an attention layer sees of its cache during one step."""
    k_pages: torch.Tensor
    v_pages: torch.Tensor
    block_table: torch.Tensor       # device int32 [max_slots, max_blocks]
    page_size: int
    window: Optional[int]
    writes: bool
    group: int


class _NoFence:
    """Stands in for a CUDA event where copies are synchronous (the CPU device of the manager's tests)."""

    def record(self):
        pass

    def synchronize(self):
        pass


class CacheGroup:
    RING = 3          # staging snapshots in flight: one per step the host may run ahead of the device, and one to spare

    def __init__(self, index, request, cache_ids, num_pages, page_size, max_slots, max_blocks, dtype, device):
        self.index, self.request, self.cache_ids = index, request, list(cache_ids)
        self.page_size, self.window = page_size, request.window
        self.pool = PagePool(num_pages)
        self.tables = [[] for _ in range(max_slots)]       # per slot: page of each logical block, or -1
        self.first_block = [0] * max_slots                 # blocks before this were given back
        shape = (num_pages, page_size, request.kv_heads, request.head_dim)
        self.k = {c: torch.zeros(shape, dtype=dtype, device=device) for c in cache_ids}
        self.v = {c: torch.zeros(shape, dtype=dtype, device=device) for c in cache_ids}
        pin = torch.device(device).type == "cuda"
        self.host_table = torch.full((max_slots, max_blocks), -1, dtype=torch.int32)      # the live table
        self.host_view = self.host_table.numpy()           # the same memory: single entries are written through this
        self.device_table = torch.full((max_slots, max_blocks), -1, dtype=torch.int32, device=device)
        self.dirty = {}                                    # slot -> (lo, hi) block range to copy
        # what the asynchronous copies read: snapshots of the dirty ranges, taken at flush()
        self._staging = [torch.empty(max_slots * max_blocks, dtype=torch.int32, pin_memory=pin) for _ in range(self.RING)]
        self._staging_views = [t.numpy() for t in self._staging]
        self._fences = [torch.cuda.Event() if pin else _NoFence() for _ in range(self.RING)]
        self._turn = 0

    def _mark(self, slot, block):
        lo, hi = self.dirty.get(slot, (block, block + 1))
        self.dirty[slot] = (min(lo, block), max(hi, block + 1))

    def pages_needed(self, slot, start, end):
        """(blocks to allocate, blocks to give back, first block kept) for positions [start, end).
        The blocks of a slot's table from `first_block` on are all present (blocks are only ever given
        back from the front, and allocated without gaps), so only the table's ends are looked at: a
        decode step costs the same whatever the context length."""
        ps = self.page_size
        table = self.tables[slot]
        n, first = len(table), self.first_block[slot]
        keep_from = 0
        if self.window is not None:
            keep_from = max(0, start - self.window + 1) // ps
        give_back = [b for b in range(first, min(keep_from, n)) if table[b] >= 0]
        last = (end - 1) // ps
        allocate = [b for b in range(keep_from, min(first, last + 1))]        # given back earlier, wanted again
        allocate += [b for b in range(max(keep_from, n), last + 1)]           # beyond the table's end
        return allocate, give_back, keep_from

    def pages_needed_by_scan(self, slot, start, end):
        """The same by looking at every block (what `check` compares `pages_needed` with)."""
        ps = self.page_size
        table = self.tables[slot]
        keep_from = 0
        if self.window is not None:
            keep_from = max(0, start - self.window + 1) // ps
        give_back = [b for b in range(self.first_block[slot], min(keep_from, len(table))) if table[b] >= 0]
        last = (end - 1) // ps
        allocate = [b for b in range(max(keep_from, 0), last + 1) if b >= len(table) or table[b] < 0]
        return allocate, give_back, keep_from

    def apply(self, slot, allocate, give_back, keep_from):
        table = self.tables[slot]
        for b in give_back:
            self.pool.release(table[b])
            table[b] = -1
            self.host_view[slot, b] = -1
            self._mark(slot, b)
        self.first_block[slot] = max(self.first_block[slot], min(keep_from, len(table)))
        for b in allocate:
            while len(table) <= b:
                table.append(-1)
            page = self.pool.allocate()
            table[b] = page
            self.host_view[slot, b] = page
            self._mark(slot, b)

    def release_slot(self, slot):
        table = self.tables[slot]
        for b, page in enumerate(table):
            if page >= 0:
                self.pool.release(page)
        if table:
            self.host_view[slot, :len(table)] = -1
            self.dirty[slot] = (0, max(len(table), self.dirty.get(slot, (0, 0))[1]))
        self.tables[slot] = []
        self.first_block[slot] = 0

    def held_pages(self):
        return [p for table in self.tables for p in table if p >= 0]

    @staticmethod
    def _copy(destination, source):
        destination.copy_(source, non_blocking=True)

    def flush(self):
        if not self.dirty:
            return
        self._turn = (self._turn + 1) % self.RING
        staging, view, fence = self._staging[self._turn], self._staging_views[self._turn], self._fences[self._turn]
        fence.synchronize()                                # the copies that read this buffer last have run
        at = 0
        for slot, (lo, hi) in self.dirty.items():
            count = hi - lo
            view[at:at + count] = self.host_view[slot, lo:hi]
            self._copy(self.device_table[slot, lo:hi], staging[at:at + count])
            at += count
        fence.record()
        self.dirty = {}


class CacheManager:
    """`cache_requests`: cache id -> KVCacheRequest; `state_requests`: state id -> StateRequest.
    `num_pages` pages of `page_size` tokens per group; `max_context` bounds a request's positions."""

    def __init__(self, cache_requests: dict, state_requests: dict, num_pages: int, page_size: int,
                 max_slots: int, max_context: int, dtype: torch.dtype, device="cpu"):
        if page_size <= 0 or max_slots <= 0 or max_context <= 0:
            raise PageError("page_size, max_slots and max_context must be positive")
        self.page_size, self.max_slots, self.max_context = page_size, max_slots, max_context
        self.max_blocks = (max_context + page_size - 1) // page_size
        self.device = device
        by_need = {}
        for cache_id, request in sorted(cache_requests.items()):
            by_need.setdefault(request, []).append(cache_id)
        self.groups = [CacheGroup(i, request, ids, num_pages, page_size, max_slots, self.max_blocks, dtype, device)
                       for i, (request, ids) in enumerate(by_need.items())]
        self.group_of = {c: g for g in self.groups for c in g.cache_ids}
        self.states = {sid: torch.zeros((max_slots, *req.shape), dtype=req.dtype, device=device)
                       for sid, req in state_requests.items()}
        self._free_slots = list(range(max_slots - 1, -1, -1))
        self._live = set()
        self.length = [0] * max_slots          # positions [0, length) have been ensured

    # ---- slots ----
    def free_slots(self) -> int:
        return len(self._free_slots)

    def live_slots(self):
        return sorted(self._live)

    def admit(self) -> int:
        """Take a slot for a new request; its state is zeroed.  Raises when none is free."""
        if not self._free_slots:
            raise PageError("no free request slot")
        slot = self._free_slots.pop()
        self._live.add(slot)
        self.length[slot] = 0
        for state in self.states.values():
            state[slot].zero_()
        return slot

    def release(self, slot: int) -> None:
        if slot not in self._live:
            raise PageError(f"slot {slot} released twice or never admitted")
        for group in self.groups:
            group.release_slot(slot)
        self._live.remove(slot)
        self._free_slots.append(slot)
        self.length[slot] = 0

    # ---- pages ----
    def available_pages(self) -> int:
        """Free pages of the tightest group."""
        return min((g.pool.available() for g in self.groups), default=1 << 30)

    def pages_for(self, slot: int, start: int, end: int) -> int:
        """How many free pages `ensure(slot, start, end)` would need in the tightest group,
        counting the pages it would first give back."""
        if all(group.window is None and (end - 1) // group.page_size < len(group.tables[slot]) for group in self.groups):
            return 0                                              # every position already has its page
        worst = 0
        for group in self.groups:
            allocate, give_back, _ = group.pages_needed(slot, start, end)
            worst = max(worst, len(allocate) - len(give_back))
        return worst

    def ensure(self, slot: int, start: int, end: int) -> bool:
        """Make pages present for positions [start, end) of `slot` in every group, all or nothing.
        False: some group has too few free pages (nothing was changed)."""
        if slot not in self._live:
            raise PageError(f"slot {slot} is not live")
        if not 0 <= start < end or end > self.max_context:
            raise PageError(f"positions [{start}, {end}) are outside the context of {self.max_context}")
        if all(group.window is None and (end - 1) // group.page_size < len(group.tables[slot]) for group in self.groups):
            self.length[slot] = max(self.length[slot], end)      # every position already has its page (most decode steps)
            return True
        plans = []
        for group in self.groups:
            allocate, give_back, keep_from = group.pages_needed(slot, start, end)
            if len(allocate) - len(give_back) > group.pool.available():
                return False
            plans.append((group, allocate, give_back, keep_from))
        for group, allocate, give_back, keep_from in plans:
            group.apply(slot, allocate, give_back, keep_from)
        self.length[slot] = max(self.length[slot], end)
        return True

    def flush(self) -> None:
        """Copy changed block-table rows to the device (asynchronous from pinned memory)."""
        for group in self.groups:
            group.flush()

    def kv_view(self, cache_id: int, writes: bool) -> KVView:
        group = self.group_of[cache_id]
        return KVView(group.k[cache_id], group.v[cache_id], group.device_table, group.page_size,
                      group.window, writes, group.index)

    def state(self, state_id):
        return self.states.get(state_id)

    def check(self) -> None:
        """Assert the invariants: no page lost, none held twice, none both free and held."""
        for group in self.groups:
            held = group.held_pages()
            if len(set(held)) != len(held):
                raise PageError(f"group {group.index}: a page is held twice")
            group.pool.check(held)
            for slot in self._live:                          # the table's shape that pages_needed relies on
                table, first = group.tables[slot], group.first_block[slot]
                if any(p >= 0 for p in table[:first]) or any(p < 0 for p in table[first:]):
                    raise PageError(f"group {group.index}, slot {slot}: the block table has a gap")
                probe = (self.length[slot], self.length[slot] + 1)
                if self.length[slot] < self.max_context and \
                        group.pages_needed(slot, *probe) != group.pages_needed_by_scan(slot, *probe):
                    raise PageError(f"group {group.index}, slot {slot}: pages_needed disagrees with a scan of the table")
        if len(set(self._free_slots)) != len(self._free_slots) or set(self._free_slots) & self._live:
            raise PageError("a slot is both free and live, or free twice")
        if len(self._free_slots) + len(self._live) != self.max_slots:
            raise PageError("a slot was lost")
