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


def plain_staging(entries, reserved, vocab, max_batch_tokens, pad_above=8, pad_to=8):
    """The step's metadata as plain Python writes it (the oracle of the native staging): returns (words, rows of
    the batch, wanted rows, rows of nobody, rows of single tokens, portions) or the refusal's message."""
    out_rows, rows, seen, n = [], [], set(), 0
    for (slot, tokens, start, want), upto in zip(entries, reserved):
        count = len(tokens)
        if count == 0:
            return "a step entry brings no tokens"
        if slot in seen:
            return f"request slot {slot} appears twice in one step"
        seen.add(slot)
        if upto < 0:
            return f"request slot {slot} is not live"
        if start < 0 or start + count > upto:
            return f"slot {slot}: positions [{start}, {start + count}) have no reserved pages (reserved up to {upto})"
        if min(tokens) < 0 or max(tokens) >= vocab:
            return f"token id {min(tokens) if min(tokens) < 0 else max(tokens)} is outside the vocabulary of {vocab}"
        for w in want:
            if not 0 <= w < count:
                return f"wanted index {w} is outside the entry's {count} tokens"
            out_rows.append(n + w)
        rows.append((slot, start, count, n, tokens))
        n += count
    if n > max_batch_tokens:
        return f"{n} tokens in one step exceed max_batch_tokens={max_batch_tokens}"
    padding = 0
    if len(rows) == n and n > pad_above and (n + pad_to - 1) // pad_to * pad_to <= max_batch_tokens:
        padding = (n + pad_to - 1) // pad_to * pad_to - n
    token_part = [t for _, _, _, _, tokens in rows for t in tokens] + [0] * padding
    position_part = [start + i for _, start, count, _, _ in rows for i in range(count)] + [0] * padding
    slot_part = [slot for slot, _, count, _, _ in rows for _ in range(count)] + [-1] * padding
    out_rows += list(range(n, n + padding))
    singles = [offset for _, _, count, offset, _ in rows if count == 1] + list(range(n, n + padding))
    portion_rows = [offset + i for _, _, count, offset, _ in rows if count > 1 for i in range(count)]
    portions = [x for _, start, count, offset, _ in rows if count > 1 for x in (offset, start, count)]
    words = token_part + position_part + slot_part + out_rows + singles + portion_rows + portions
    return words, n + padding, len(out_rows), padding, len(singles), len(portions) // 3


@pytest.mark.parametrize("seed", range(6))
def test_native_staging_of_a_step_against_plain_python(seed):
    """Random batches, good ones and ones with every kind of fault, through the native staging of the step function
    (csrc/host/step_host.cpp) and through plain Python: the same words, the same counts, the same refusals."""
    import ctypes

    import numpy as np
    from lia_rs_b200.cache.pages import host_library
    rng = random.Random(seed)
    lib = host_library()
    m = manager(num_pages=400, page_size=4, max_slots=24)
    lengths = {}
    for _ in range(rng.randint(4, 20)):
        slot = m.admit()
        lengths[slot] = rng.randint(1, 60)
        assert m.ensure(slot, 0, lengths[slot])
    vocab, budget = 97, 96
    meta = np.full(7 * budget, -7, dtype=np.int32)
    summary = (ctypes.c_int * 8)()
    refusals = 0
    for trial in range(300):
        chosen = rng.sample(sorted(lengths), rng.randint(1, len(lengths)))
        singles_only = rng.random() < 0.5
        entries = []
        for slot in chosen:
            count = 1 if singles_only else rng.randint(1, min(12, lengths[slot]))
            start = rng.randint(0, lengths[slot] - count)
            want = sorted(rng.sample(range(count), rng.randint(0, min(count, 2))))
            entries.append([slot, [rng.randrange(vocab) for _ in range(count)], start, want])
        fault = rng.randrange(12)
        victim = rng.randrange(len(entries))
        if fault == 0:
            entries[victim][1] = []
        elif fault == 1 and len(entries) > 1:
            entries[victim][0] = entries[victim - 1][0]
        elif fault == 2:
            entries[victim][0] = rng.choice([-1, 24, 23 if 23 not in lengths else 99])
        elif fault == 3:
            entries[victim][2] = lengths[entries[victim][0]] - len(entries[victim][1]) + 1
        elif fault == 4:
            entries[victim][1][rng.randrange(len(entries[victim][1]))] = rng.choice([-1, vocab, 10**6])
        elif fault == 5:
            entries[victim][3] = [len(entries[victim][1])]
        reserved = m.reserved([e[0] for e in entries])
        expected = plain_staging(entries, reserved, vocab, budget)
        n_entries = len(entries)
        Entries = ctypes.c_int * n_entries
        tokens = [t for e in entries for t in e[1]]
        wants = [w for e in entries for w in e[3]]
        meta[:] = -7
        rc = lib.lia_step_stage(m.native_handle(), n_entries, Entries(*[e[0] for e in entries]), Entries(*[e[2] for e in entries]),
                                Entries(*[len(e[1]) for e in entries]), (ctypes.c_int * max(1, len(tokens)))(*tokens),
                                Entries(*[len(e[3]) for e in entries]), (ctypes.c_int * max(1, len(wants)))(*wants), vocab, budget,
                                8, 8, ctypes.c_void_p(meta.ctypes.data), ctypes.c_longlong(meta.size), summary)
        if isinstance(expected, str):
            refusals += 1
            assert rc < 0 and lib.lia_host_error().decode() == expected
            continue
        words, n, n_out, padding, n_single, n_portions = expected
        assert rc == 0, lib.lia_host_error().decode()
        assert list(summary[:6]) == [n, n_out, padding, n_single, n_portions, len(words)]
        assert meta[:len(words)].tolist() == words and (meta[len(words):] == -7).all()
    assert 60 < refusals < 250
