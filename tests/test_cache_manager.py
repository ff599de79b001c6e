"""The cache manager on the CPU: no page lost, held twice or freed twice, under random orders of
requests; windows give pages back; slots of per-request state."""
import random

import pytest
import torch

from lia_rs_b200.cache import CacheManager, PageError, PagePool
from lia_rs_b200.parts import KVCacheRequest, StateRequest


def manager(num_pages=12, page_size=4, max_slots=4, window=None, two_groups=False, states=None):
    requests = {0: KVCacheRequest(2, 16, window), 1: KVCacheRequest(2, 16, window)}
    if two_groups:
        requests[2] = KVCacheRequest(2, 16, None if window else 6)
    return CacheManager(requests, states or {}, num_pages, page_size, max_slots, 256, torch.float32, "cpu")


def test_pool_refuses_double_free_and_exhaustion():
    pool = PagePool(2)
    a, b = pool.allocate(), pool.allocate()
    assert {a, b} == {0, 1} and pool.available() == 0
    with pytest.raises(PageError, match="exhausted"):
        pool.allocate()
    pool.release(a)
    with pytest.raises(PageError, match="freed twice"):
        pool.release(a)
    assert pool.allocate() == a          # the page given back is used again first
    with pytest.raises(PageError, match="outside"):
        pool.release(7)


def test_ensure_is_all_or_nothing_and_tables_follow():
    m = manager(num_pages=5)
    s = m.admit()
    assert m.ensure(s, 0, 9) and m.groups[0].pool.in_use() == 3
    assert m.groups[0].tables[s] == [0, 1, 2]
    assert not m.ensure(s, 9, 30)                     # needs 5 more pages, 2 are free
    assert m.groups[0].pool.in_use() == 3 and m.length[s] == 9
    assert m.ensure(s, 9, 20) and m.groups[0].pool.available() == 0
    m.flush()
    assert m.groups[0].device_table[s, :5].tolist() == m.groups[0].tables[s]
    assert m.groups[0].device_table[s, 5].item() == -1
    m.check()
    m.release(s)
    m.flush()
    assert m.groups[0].device_table[s, :5].tolist() == [-1] * 5 and m.groups[0].pool.in_use() == 0
    with pytest.raises(PageError, match="released twice"):
        m.release(s)
    with pytest.raises(PageError, match="outside the context"):
        m.ensure(m.admit(), 250, 300)


def test_layers_of_one_need_share_a_group_and_kv_views():
    m = manager(two_groups=True)
    assert len(m.groups) == 2 and m.groups[0].cache_ids == [0, 1] and m.groups[1].cache_ids == [2]
    view = m.kv_view(1, True)
    assert view.k_pages.shape == (12, 4, 2, 16) and view.block_table is m.groups[0].device_table
    assert m.kv_view(2, False).window == 6 and not m.kv_view(2, False).writes


def test_window_gives_pages_back_once_passed():
    m = manager(num_pages=6, page_size=4, window=6)
    s = m.admit()
    assert m.ensure(s, 0, 10)                          # blocks 0..2
    assert m.groups[0].pool.in_use() == 3
    assert m.ensure(s, 10, 11)                         # keys 5..10 visible: block 0 (0..3) is passed
    assert m.groups[0].tables[s][:3] == [-1, 1, 2] and m.groups[0].pool.in_use() == 2
    for pos in range(11, 60):
        assert m.ensure(s, pos, pos + 1)
        assert m.groups[0].pool.in_use() <= 3          # a window of 6 never holds more than 3 pages of 4
        m.check()
    # a long portion needs the pages of its whole span at once
    assert not m.ensure(s, 60, 80)                      # keys 55..79 span 7 pages
    assert m.ensure(s, 60, 76) and m.groups[0].pool.in_use() == 6
    m.release(s)
    m.check()


def test_state_slots_are_zeroed_on_admission():
    m = manager(states={5: StateRequest((3, 2), torch.float32)})
    s = m.admit()
    assert m.state(5).shape == (4, 3, 2) and m.state(4) is None
    m.state(5)[s] += 7
    m.release(s)
    assert m.admit() == s and float(m.state(5)[s].abs().sum()) == 0.0


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_of_requests(seed):
    rng = random.Random(seed)
    m = manager(num_pages=rng.choice([6, 9, 16]), page_size=rng.choice([2, 4, 8]),
                window=rng.choice([None, 5, 13]), two_groups=rng.random() < 0.5)
    live = {}
    for _ in range(400):
        action = rng.random()
        if action < 0.25 and m.free_slots():
            live[m.admit()] = 0
        elif action < 0.85 and live:
            slot = rng.choice(list(live))
            count = rng.choice([1, 1, 1, 2, 5, 9])
            if live[slot] + count <= 256:
                before = [g.pool.in_use() for g in m.groups]
                if m.ensure(slot, live[slot], live[slot] + count):
                    live[slot] += count
                else:
                    assert before == [g.pool.in_use() for g in m.groups]
        elif live:
            slot = rng.choice(list(live))
            m.release(slot)
            del live[slot]
        m.check()
        for group in m.groups:
            for slot, length in live.items():
                first = 0 if group.window is None else max(0, length - group.window)
                for pos in range(first, length):       # every position that can still be seen has a page
                    assert group.tables[slot][pos // m.page_size] >= 0
    for slot in list(live):
        m.release(slot)
    m.check()
    assert all(g.pool.in_use() == 0 for g in m.groups) and m.free_slots() == 4


class DeferredDevice:
    """A stand-in for the stream: copies queued by `flush` run only when asked to (or when a fence that was
    recorded after them is waited for), and they read their source THEN, as an asynchronous copy does."""

    def __init__(self):
        self.queue = []          # ("copy", destination, source) | ("fence", fence)

    def copy(self, destination, source):
        self.queue.append(("copy", destination, source))

    def fence(self):
        device = self

        class Fence:
            recorded = False

            def record(self):
                self.recorded = True
                device.queue.append(("fence", self))

            def synchronize(self):
                if self.recorded and any(item[0] == "fence" and item[1] is self for item in device.queue):
                    device.run_until(self)
        return Fence()

    def run_until(self, fence=None):
        while self.queue:
            item = self.queue.pop(0)
            if item[0] == "copy":
                item[1].copy_(item[2])
            elif item[1] is fence:
                return


def deferred(m):
    device = DeferredDevice()
    for group in m.groups:
        group._copy = device.copy
        group._fences = [device.fence() for _ in group._fences]
    return device


def test_queued_table_copies_see_the_table_of_flush_time_whatever_the_host_does_next():
    """The pipelined scheduler flushes for step N+1, then learns that a request of step N ended and releases
    it, which resets its row on the host, before the queued copy has run.  The device must still receive the
    row as it was at the flush: the step that is queued holds the request."""
    m = manager(num_pages=12)
    device = deferred(m)
    a, b = m.admit(), m.admit()
    assert m.ensure(a, 0, 9) and m.ensure(b, 0, 5)
    at_flush = {a: list(m.groups[0].tables[a]), b: list(m.groups[0].tables[b])}
    m.flush()                                   # copies are queued, none has run
    m.release(a)                                # the host resets a's row (and would hand its pages to others)
    assert m.ensure(b, 5, 13)                   # b's row grows on the host
    device.run_until()                          # now the device catches up with the first flush
    table = m.groups[0].device_table
    assert table[a, :3].tolist() == at_flush[a], "the queued copy read the live table"
    assert table[b, :2].tolist() == at_flush[b] and table[b, 2].item() == -1
    m.flush()
    device.run_until()
    assert table[a, :3].tolist() == [-1, -1, -1] and table[b, :4].tolist() == m.groups[0].tables[b]
    m.check()


def test_staging_ring_waits_for_its_own_copies_before_it_is_written_again():
    m = manager(num_pages=40, page_size=2, max_slots=2)
    device = deferred(m)
    s = m.admit()
    seen = []
    for step in range(3 * m.groups[0].RING):    # far more flushes than staging buffers, none of them run yet
        assert m.ensure(s, 2 * step, 2 * step + 2)
        seen.append(list(m.groups[0].tables[s]))
        m.flush()
    device.run_until()
    assert m.groups[0].device_table[s, :len(seen[-1])].tolist() == seen[-1]
    m.check()
