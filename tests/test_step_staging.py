"""`StepRuntime.begin` on the CPU: the face of the native staging, with the device's buffers as CPU tensors and a
stand-in for the copy's event (the runtime itself needs pinned memory and a device)."""
import ctypes

import pytest
import torch

from lia_rs_b200.cache import CacheManager
from lia_rs_b200.cache.pages import host_library
from lia_rs_b200.engine.step import StepEntry, StepError, StepRuntime
from lia_rs_b200.parts import KVCacheRequest


class _Event:
    def synchronize(self):
        pass

    def record(self):
        pass


def cpu_runtime(max_batch_tokens=32, max_slots=12, vocab=50):
    cache = CacheManager({0: KVCacheRequest(2, 16, None)}, {}, 200, 4, max_slots, 256, torch.float32, "cpu")
    runtime = object.__new__(StepRuntime)
    runtime.cache, runtime.vocab_size, runtime.max_batch_tokens = cache, vocab, max_batch_tokens
    runtime.device = torch.device("cpu")
    runtime._meta_host = torch.zeros(7 * max_batch_tokens, dtype=torch.int32)
    runtime._meta_view = runtime._meta_host.numpy()
    runtime._meta_device = torch.full((7 * max_batch_tokens,), -9, dtype=torch.int32)
    runtime.error_flag = torch.zeros(1, dtype=torch.int32)
    runtime._error_host = torch.zeros(1, dtype=torch.int32)
    runtime._copy_event = _Event()
    runtime._host, runtime._summary = host_library(), (ctypes.c_int * 8)()
    runtime._buffers, runtime._attentions = {}, {}
    return runtime, cache


def test_a_mixed_step_is_laid_out_for_the_kernels():
    runtime, cache = cpu_runtime()
    a, b, c = cache.admit(), cache.admit(), cache.admit()
    for slot, upto in ((a, 20), (b, 9), (c, 6)):
        assert cache.ensure(slot, 0, upto)
    ctx = runtime.begin([StepEntry(a, [7], 19, [0]), StepEntry(b, [1, 2, 3, 4], 5, [0, 3]), StepEntry(c, [9], 2, [])])
    assert (ctx.n_tokens, ctx.n_out, ctx.padding, ctx.n_single, ctx.n_prefill_segments) == (6, 3, 0, 2, 1)
    assert ctx.segments == [(a, 19, 1, 0), (b, 5, 4, 1), (c, 2, 1, 5)]
    assert ctx.tokens.tolist() == [7, 1, 2, 3, 4, 9]
    assert ctx.positions.tolist() == [19, 5, 6, 7, 8, 2]
    assert ctx.slots.tolist() == [a, b, b, b, b, c]
    assert ctx.out_rows.tolist() == [0, 1, 4]
    assert ctx.decode_rows.tolist() == [0, 5] and ctx.prefill_rows.tolist() == [1, 2, 3, 4]
    assert ctx.prefill_segments.tolist() == [1, 5, 4]
    assert not ctx.decode_only and ctx.max_context == 20 and runtime.h2d_bytes == 4 * (4 * 6 + 3 + 3)


def test_single_tokens_beyond_eight_get_rows_of_nobody_and_fed_tokens_go_to_the_real_rows_only():
    runtime, cache = cpu_runtime()
    slots = [cache.admit() for _ in range(10)]
    for slot in slots:
        assert cache.ensure(slot, 0, 5)
    feed = torch.arange(100, 116, dtype=torch.int32)
    ctx = runtime.begin([StepEntry(slot, [0], 4, [0]) for slot in slots], feed=feed)
    assert (ctx.n_tokens, ctx.n_out, ctx.padding, ctx.n_single) == (16, 16, 6, 16) and len(ctx.segments) == 10
    assert ctx.tokens.tolist() == list(range(100, 110)) + [0] * 6
    assert ctx.slots.tolist() == slots + [-1] * 6 and ctx.positions.tolist() == [4] * 10 + [0] * 6
    assert ctx.out_rows.tolist() == list(range(16)) == ctx.decode_rows.tolist()
    assert ctx.decode_only and ctx.prefill_rows.numel() == 0 and ctx.prefill_segments.numel() == 0
    with pytest.raises(StepError, match="only to a step of single tokens"):
        runtime.begin([StepEntry(slots[0], [1, 2], 3, [])], feed=feed)


def test_refusals_carry_the_native_message_and_numbers_that_do_not_fit():
    runtime, cache = cpu_runtime()
    slot = cache.admit()
    assert cache.ensure(slot, 0, 8)
    for entries, message in (([StepEntry(slot, [], 0)], "brings no tokens"),
                             ([StepEntry(slot, [1], 0), StepEntry(slot, [2], 1)], "appears twice"),
                             ([StepEntry(5, [1], 0)], "is not live"),
                             ([StepEntry(slot, [1, 2], 7)], "no reserved pages"),
                             ([StepEntry(slot, [1, 50], 0)], "token id 50 is outside the vocabulary of 50"),
                             ([StepEntry(slot, [10**12], 0)], "token id 1000000000000 is outside the vocabulary"),
                             ([StepEntry(slot, [1], 0, [1])], "wanted index 1"),
                             ([StepEntry(slot, [1], 2**32, [0])], "must fit 32 bits"),
                             ([StepEntry(slot, [1], 0, [None])], "must be integers"),
                             ([StepEntry(slot, [1] * 33, 0)], "no reserved pages")):
        with pytest.raises(StepError, match=message):
            runtime.begin(entries)
    assert cache.ensure(slot, 0, 40)
    with pytest.raises(StepError, match="33 tokens in one step exceed max_batch_tokens=32"):
        runtime.begin([StepEntry(slot, [1] * 33, 0)])
    ctx = runtime.begin([StepEntry(slot, [3, 4], 0, [1])])          # and the runtime is as good as before
    assert ctx.tokens.tolist() == [3, 4] and ctx.out_rows.tolist() == [1]
