"""Failures made on the host, and the engine afterwards: every refusal of a step's host checks, the device's
error flag for a token id out of range, for a block-table row without a page and for a bounded wait that
runs out, each followed by a good step with the right logits; an end of sequence at a page's edge inside a
pipelined run.  No test here faults, traps or hangs the GPU: the flags are raised by kernels that skip the
bad access and return.

The reference fails every job on a step error and stays consistent (src/server/paged.rs:85-98); its host
checks are src/inference/paging.rs:120-172."""
import numpy as np
import pytest
import torch

import helpers
import plain_impl

pytestmark = pytest.mark.gpu


def make_engine(model, dtype="float32", **options):
    from lia_rs_b200.engine import Engine
    return Engine(model["dir"], dtype=dtype, page_size=model["page_size"], max_tokens=256, max_seqs=4,
                  max_batch_tokens=64, **options)


def good_step(engine, model, dtype, what):
    """A fresh request whole, against the plain implementation."""
    tokens = helpers.random_tokens(model["config"]["vocab_size"], 23, 9)
    replay = helpers.Replayer(engine)
    logits = replay.step([("good", tokens, range(len(tokens)))], end=["good"])
    helpers.assert_close(logits, helpers.plain_logits(model, tokens, dtype), dtype, what)


def test_every_host_refusal_leaves_the_engine_usable(tiny_models):
    from lia_rs_b200.engine import StepEntry, StepError
    model = tiny_models["tiny-B"]
    vocab = model["config"]["vocab_size"]
    engine = make_engine(model)
    slot = engine.admit()
    assert engine.reserve(slot, 0, 8)
    free = engine.cache.free_slots()
    cases = [
        ([StepEntry(slot, [], 0)], "brings no tokens"),
        ([StepEntry(slot, [1, 2], 0), StepEntry(slot, [3], 2)], "appears twice"),
        ([StepEntry(3, [1], 0)], "is not live"),
        ([StepEntry(slot, [1] * 9, 0)], "no reserved pages"),
        ([StepEntry(slot, [1, 2], 7)], "no reserved pages"),
        ([StepEntry(slot, [1, vocab], 0)], "outside the vocabulary"),
        ([StepEntry(slot, [-1], 0)], "outside the vocabulary"),
        ([StepEntry(slot, [1, 2], 0, want=[2])], "wanted index"),
    ]
    for entries, message in cases:
        with pytest.raises(StepError, match=message):
            engine.step(entries)
        engine.synchronize()
        assert engine.cache.free_slots() == free
        engine.cache.check()
    other = engine.admit()
    assert engine.reserve(other, 0, 65)
    with pytest.raises(StepError, match="exceed max_batch_tokens"):
        engine.step([StepEntry(other, [1] * 65, 0)])
    engine.release(other)
    # the request that the refused steps named is still whole: its tokens go through and are right
    tokens = helpers.random_tokens(vocab, 8, 4)
    logits = engine.step([StepEntry(slot, tokens, 0, want=list(range(8)))]).cpu().numpy()
    engine.synchronize()
    helpers.assert_close(logits, helpers.plain_logits(model, tokens, "float32"), "float32", "after the refusals")
    engine.release(slot)
    good_step(engine, model, "float32", "a fresh request after the refusals")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_token_id_out_of_range_on_the_device_raises_at_the_next_synchronisation(tiny_models, dtype):
    """Ids fed on the device (the pipelined scheduler's path) pass no host check: the embedding kernel writes
    zeros for a bad one, raises flag 1, and the engine reports it; the next steps are right."""
    from lia_rs_b200.engine import StepEntry, StepError
    from lia_rs_b200.engine.engine import PendingTokens
    model = tiny_models["tiny-D"]
    vocab = model["config"]["vocab_size"]
    engine = make_engine(model, dtype)
    slot = engine.admit()
    assert engine.reserve(slot, 0, 2)
    engine.step([StepEntry(slot, [5], 0, want=[0])])
    bad = torch.tensor([vocab + 7], dtype=torch.int32, device=engine.device)
    feed = PendingTokens(engine, bad, None, None)
    engine.step([StepEntry(slot, [0], 1, want=[0])], feed=feed)
    with pytest.raises(StepError, match="outside the vocabulary"):
        engine.synchronize()
    engine.synchronize()                                  # raised once, then clear
    engine.release(slot)
    good_step(engine, model, dtype, "after a bad id on the device")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tokens_in_step", [1, 5])
def test_a_table_row_without_a_page_raises_and_reads_nothing_outside_the_pool(tiny_models, dtype, tokens_in_step):
    """The test blanks a request's block-table row on the device (what a lost copy would leave): the append and
    every attention kernel skip the missing page, raise flag 2, and the engine reports it."""
    from lia_rs_b200.engine import StepEntry, StepError
    model = tiny_models["tiny-E"]
    vocab = model["config"]["vocab_size"]
    engine = make_engine(model, dtype)
    slot = engine.admit()
    prompt = helpers.random_tokens(vocab, 30, 3)
    assert engine.reserve(slot, 0, 30 + tokens_in_step)
    engine.step([StepEntry(slot, prompt, 0)])
    engine.synchronize()
    for group in engine.cache.groups:
        group.device_table[slot].fill_(-1)
    engine.step([StepEntry(slot, helpers.random_tokens(vocab, tokens_in_step, 4), 30, want=[0])])
    with pytest.raises(StepError, match="no page"):
        engine.synchronize()
    engine.release(slot)
    good_step(engine, model, dtype, "after a row without pages")


def test_a_bounded_wait_that_runs_out_is_reported_and_the_next_product_is_right(tiny_models):
    """A kernel waits on an mbarrier at which nobody arrives, gives up after 3,000 polls and raises flag 3, as the
    tensor-core kernels' waits would: the engine reports it, zeroes the counters that a kernel that gave up may
    have left mid-count, and goes on."""
    from lia_rs_b200.engine import StepError
    from lia_rs_b200.kernels import ops
    model = tiny_models["tiny-D"]
    engine = make_engine(model, "bfloat16")
    good_step(engine, model, "bfloat16", "before")
    gave_up = torch.zeros(1, dtype=torch.int32, device=engine.device)
    scratch, _ = ops._device_scratch(engine.device)
    scratch[:4].fill_(1.0)                                # as if a split-K product had stopped mid-count
    ops.wait_probe(3000, engine.runtime_step.error_flag, gave_up)
    engine.runtime_step.finish()
    with pytest.raises(StepError, match="gave up waiting"):
        engine.synchronize()
    assert gave_up.item() == 1
    assert float(scratch[:ops.COUNTER_WORDS].abs().sum()) == 0.0
    good_step(engine, model, "bfloat16", "after a wait that ran out")
    # and a split-K product on its own
    torch.manual_seed(0)
    a = torch.randn(8, 2048, device=engine.device).to(torch.bfloat16)
    w = (torch.randn(2560, 2048, device=engine.device) / 45.0).to(torch.bfloat16)
    out = torch.empty(8, 2560, device=engine.device)
    flag = torch.zeros(1, dtype=torch.int32, device=engine.device)
    ops.gemm_tc(ops.GEMM_STORE, a, w, out, 1.0, flag)
    exact = a.double() @ w.double().T
    assert float((out.double() - exact).abs().max()) < 2e-5 * max(1.0, float(exact.abs().max())) * (2048 / 64) ** 0.5
    assert flag.item() == 0


def test_end_of_sequence_at_a_page_edge_inside_a_pipelined_run(tiny_models):
    """A request is ended by its token just as the step that was launched ahead of it (with the token fed on the
    device) took a new page for it; the others decode on.  Tokens equal the plain implementation's, pages and
    slots all come back."""
    from lia_rs_b200.engine.generate import Generator
    model = tiny_models["tiny-B"]
    vocab, page = model["config"]["vocab_size"], model["page_size"]
    prompts = [helpers.random_tokens(vocab, n, 300 + n) for n in (9, 14, 21)]
    full = [plain_impl.greedy(model["config"], model["weights"], p, 40) for p in prompts]
    assert all(len(set(tokens)) > 3 for tokens in full), "the model's greedy output is not degenerate"
    # a token that some request produces for the first time just where feeding it back opens a new page: the step
    # launched ahead has reserved that page when the host reads the token and ends the request
    eos = None
    for tokens, prompt in zip(full, prompts):
        for j in range(2, 31):
            if (len(prompt) + j) % page == 0 and tokens[j] not in tokens[:j]:
                eos = tokens[j]
    assert eos is not None
    want = []
    for tokens in full:
        cut = tokens.index(eos) + 1 if eos in tokens else len(tokens)
        want.append(tokens[:cut])
    generator = Generator(model["dir"], dtype="float32", page_size=page, kv_pool_tokens=512, max_sequences=4,
                          prefill_batch=64)
    got = generator.generate(prompts, max_tokens=40, eos_token_ids=[eos])
    assert got == want
    assert generator.last_scheduler.stats["pipelined_steps"] > 10
    generator.engine.cache.check()
    assert generator.engine.cache.free_slots() == 4
    assert all(group.pool.in_use() == 0 for group in generator.engine.cache.groups)
