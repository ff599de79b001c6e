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

The bookkeeping (pools, the tables of every slot, what an `ensure` has to allocate and give back, which table
rows changed) is native: csrc/host/cache_host.cpp, one object for all groups of a manager; the classes here are
its faces and own the tensors.  The manager runs on the CPU device too, which is how its tests exercise it
without a GPU.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import ctypes

import torch

from .pages import PageError, host_library, raise_last


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


class _PoolFace:
    """What `group.pool` answers: the pool of one group of the native cache."""

    def __init__(self, group):
        self._group = group
        self.num_pages = group.num_pages

    def available(self) -> int:
        return self._group._lib.lia_cache_available(self._group._native(), self._group.index)

    def in_use(self) -> int:
        return self.num_pages - self.available()


class _Tables:
    """`group.tables[slot]`: the page of each logical block of the slot (a list; -1: given back)."""

    def __init__(self, group):
        self._group = group

    def __getitem__(self, slot):
        group = self._group
        out = (ctypes.c_int * group.max_blocks)()
        n = group._lib.lia_cache_table(group._native(), group.index, int(slot), out, group.max_blocks)
        if n < 0:
            raise_last()
        return list(out[:n])

    def __len__(self):
        return self._group.max_slots

    def __iter__(self):
        return (self[slot] for slot in range(self._group.max_slots))


class _FirstBlocks:
    def __init__(self, group):
        self._group = group

    def __getitem__(self, slot):
        return self._group._lib.lia_cache_first_block(self._group._native(), self._group.index, int(slot))


class CacheGroup:
    RING = 3          # staging snapshots in flight: one per step the host may run ahead of the device, and one to spare

    def __init__(self, index, request, cache_ids, num_pages, page_size, max_slots, max_blocks, dtype, device):
        self.index, self.request, self.cache_ids = index, request, list(cache_ids)
        self.page_size, self.window = page_size, request.window
        self.num_pages, self.max_slots, self.max_blocks = num_pages, max_slots, max_blocks
        self._lib = host_library()
        self._owner = None                                 # the manager, which holds the native cache of all its groups
        self.pool = _PoolFace(self)
        self.tables = _Tables(self)                        # per slot: page of each logical block, or -1
        self.first_block = _FirstBlocks(self)              # blocks before this were given back
        shape = (num_pages, page_size, request.kv_heads, request.head_dim)
        self.k = {c: torch.zeros(shape, dtype=dtype, device=device) for c in cache_ids}
        self.v = {c: torch.zeros(shape, dtype=dtype, device=device) for c in cache_ids}
        pin = torch.device(device).type == "cuda"
        # the live table: the native cache writes the entries it changes straight into this memory
        self.host_table = torch.full((max_slots, max_blocks), -1, dtype=torch.int32, pin_memory=pin)
        self.host_view = self.host_table.numpy()
        self.device_table = torch.full((max_slots, max_blocks), -1, dtype=torch.int32, device=device)
        self._dirty = (ctypes.c_int * (3 * max_slots))()
        # what the asynchronous copies read: snapshots of the dirty ranges, taken at flush()
        self._staging = [torch.empty(max_slots * max_blocks, dtype=torch.int32, pin_memory=pin) for _ in range(self.RING)]
        self._staging_views = [t.numpy() for t in self._staging]
        self._fences = [torch.cuda.Event() if pin else _NoFence() for _ in range(self.RING)]
        self._turn = 0

    def _native(self):
        return self._owner._handle

    def held_pages(self):
        return [p for table in self.tables for p in table if p >= 0]

    def held_by(self, slot) -> int:
        """Pages that the slot holds in this group."""
        return self._lib.lia_cache_held(self._native(), self.index, int(slot))

    @staticmethod
    def _copy(destination, source):
        destination.copy_(source, non_blocking=True)

    def flush(self):
        n = self._lib.lia_cache_take_dirty(self._native(), self.index, self._dirty, self.max_slots)
        if n <= 0:
            return
        self._turn = (self._turn + 1) % self.RING
        staging, view, fence = self._staging[self._turn], self._staging_views[self._turn], self._fences[self._turn]
        fence.synchronize()                                # the copies that read this buffer last have run
        at = 0
        dirty = self._dirty
        for i in range(n):
            slot, lo, hi = dirty[3 * i], dirty[3 * i + 1], dirty[3 * i + 2]
            count = hi - lo
            view[at:at + count] = self.host_view[slot, lo:hi]
            self._copy(self.device_table[slot, lo:hi], staging[at:at + count])
            at += count
        fence.record()


class _Lengths:
    """`manager.length[slot]`: up to where the native cache has ensured the slot's positions."""

    def __init__(self, manager):
        self._manager = manager

    def __getitem__(self, slot: int) -> int:
        value = int(self._manager._lib.lia_cache_length(self._manager._handle, int(slot)))
        if value < 0:
            raise_last()
        return value


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
        self._lib = host_library()
        n = len(self.groups)
        IntArray, PointerArray = ctypes.c_int * max(1, n), ctypes.c_void_p * max(1, n)
        self._handle = ctypes.c_void_p(self._lib.lia_cache_create(
            n, IntArray(*[num_pages] * n), IntArray(*[page_size] * n),
            IntArray(*[-1 if g.window is None else int(g.window) for g in self.groups]), max_slots, self.max_blocks,
            PointerArray(*[g.host_table.data_ptr() for g in self.groups])))
        if not self._handle:
            raise_last()
        for group in self.groups:
            group._owner = self
        self.group_of = {c: g for g in self.groups for c in g.cache_ids}
        self.states = {sid: torch.zeros((max_slots, *req.shape), dtype=req.dtype, device=device)
                       for sid, req in state_requests.items()}
        self.length = _Lengths(self)           # positions [0, length[slot]) of a live slot have been ensured

    def __del__(self):
        handle, self._handle = getattr(self, "_handle", None), None
        if handle:
            self._lib.lia_cache_destroy(handle)

    def native_handle(self):
        """The native cache, for the host library's other entry points (the scheduler's policy, the step's staging)."""
        return self._handle

    # ---- slots (kept by the native cache: the scheduler's native policy works on the same state) ----
    def free_slots(self) -> int:
        return int(self._lib.lia_cache_free_slots(self._handle))

    def is_live(self, slot: int) -> bool:
        return bool(self._lib.lia_cache_is_live(self._handle, int(slot)))

    def reserved(self, slots) -> list:
        """For each slot: up to where it has pages, or -1 when it is not live."""
        n = len(slots)
        Array = ctypes.c_int * max(1, n)
        out = Array()
        self._lib.lia_cache_reserved(self._handle, Array(*slots), n, out)
        return out[:n]

    def live_slots(self):
        return [slot for slot in range(self.max_slots) if self.is_live(slot)]

    def admit(self) -> int:
        """Take a slot for a new request; its state is zeroed.  Raises when none is free."""
        slot = int(self._lib.lia_cache_admit(self._handle))
        if slot < 0:
            raise_last()
        self.admitted(slot)
        return slot

    def admitted(self, slot: int) -> None:
        """What the face owes a slot that the native side has just handed out: its state zeroed."""
        for state in self.states.values():
            state[slot].zero_()

    def release(self, slot: int) -> None:
        if self._lib.lia_cache_release_slot(self._handle, int(slot)) < 0:
            raise_last()

    # ---- pages ----
    def available_pages(self) -> int:
        """Free pages of the tightest group."""
        return min((g.pool.available() for g in self.groups), default=1 << 30)

    def pages_for(self, slot: int, start: int, end: int) -> int:
        """How many free pages `ensure(slot, start, end)` would need in the tightest group,
        counting the pages it would first give back."""
        worst = self._lib.lia_cache_pages_for(self._handle, int(slot), int(start), int(end))
        if worst < 0:
            raise_last()
        return worst

    def ensure(self, slot: int, start: int, end: int) -> bool:
        """Make pages present for positions [start, end) of the live slot `slot` in every group, all or nothing.
        False: some group has too few free pages (nothing was changed)."""
        done = self._lib.lia_cache_ensure(self._handle, int(slot), int(start), int(end), self.max_context)
        if done < 0:
            raise_last()
        return bool(done)

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
        live = self.live_slots()
        Array = ctypes.c_int * max(1, len(live))
        for group in self.groups:
            if self._lib.lia_cache_check(self._handle, group.index, Array(*live), Array(*[self.length[s] for s in live]),
                                         len(live), self.max_context) < 0:
                raise_last()
            # the host table (what goes to the device) says what the tables say
            for slot in live:
                table = group.tables[slot]
                if group.host_view[slot, :len(table)].tolist() != table:
                    raise PageError(f"group {group.index}, slot {slot}: the host table differs from the slot's table")
        free = (ctypes.c_int * self.max_slots)()
        free = list(free[:self._lib.lia_cache_free_slot_list(self._handle, free)])
        if len(set(free)) != len(free) or set(free) & set(live):
            raise PageError("a slot is both free and live, or free twice")
        if len(free) + len(live) != self.max_slots:
            raise PageError("a slot was lost")
