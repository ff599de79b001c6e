"""The scheduler's decisions on the CPU, with a stand-in for the engine that keeps a real cache
manager and returns logits that make the next token predictable."""
import numpy as np
import pytest
import torch

from lia_rs_b200.cache import CacheManager
from lia_rs_b200.engine.scheduler import Scheduler, SchedulerError
from lia_rs_b200.parts import KVCacheRequest
from lia_rs_b200.sampling import Sampling

VOCAB = 50


class StandInEngine:
    """next token = (sum of the request's tokens so far) mod VOCAB; records every batch and checks
    that each batch continues each request exactly where its cache ends."""

    def __init__(self, num_pages, page_size=4, max_slots=4, context=256):
        self.cache = CacheManager({0: KVCacheRequest(1, 16)}, {}, num_pages, page_size, max_slots, context,
                                  torch.float32, "cpu")
        self.seen = {}            # slot -> tokens in the cache
        self.batches = []

    def step(self, entries):
        rows = []
        self.batches.append([(e.slot, e.start, len(e.tokens), list(e.want)) for e in entries])
        for e in entries:
            have = self.seen.setdefault(e.slot, [])
            if e.start == 0:
                have.clear()
            assert e.start == len(have), "a portion does not continue where the cache ends"
            assert e.start + len(e.tokens) <= self.cache.length[e.slot], "tokens without pages"
            have.extend(e.tokens)
            for w in e.want:
                row = np.full(VOCAB, -1.0, dtype=np.float32)
                row[sum(have[:e.start + w + 1]) % VOCAB] = 1.0
                rows.append(row)
        self.cache.check()
        return torch.tensor(np.array(rows)) if rows else torch.zeros(0, VOCAB)

    def select_tokens(self, logits, samplings, positions):
        return [int(t) for t in logits.argmax(dim=-1)]

    def logits_to_host(self, logits):
        return logits.numpy()


def expected(prompt, n):
    tokens, out = list(prompt), []
    for _ in range(n):
        out.append(sum(tokens) % VOCAB)
        tokens.append(out[-1])
    return out


def test_prompts_are_cut_under_the_token_budget_and_decodes_come_first():
    engine = StandInEngine(num_pages=64)
    s = Scheduler(engine, max_batch_tokens=8)
    b = s.add("b", [7, 8, 9], max_tokens=4)
    a = s.add("a", list(range(1, 20)), max_tokens=3)
    s.run()
    assert a.generated == expected(a.prompt, 3) and b.generated == expected(b.prompt, 4)
    assert all(sum(n for _, _, n, _ in batch) <= 8 for batch in engine.batches)
    # b's whole prompt and the first 5 tokens of a fill the budget of 8
    assert engine.batches[0] == [(0, 0, 3, [2]), (1, 0, 5, [])]
    # then b decodes: its single token comes first and a's portion gets the other 7 rows
    assert engine.batches[1] == [(0, 3, 1, [0]), (1, 5, 7, [])]
    assert engine.batches[2] == [(0, 4, 1, [0]), (1, 12, 7, [6])]
    assert s.stats["prefill_tokens"] == 19 + 3 and engine.cache.available_pages() == 64


def test_even_split_gives_every_request_its_share():
    engine = StandInEngine(num_pages=64)
    s = Scheduler(engine, max_batch_tokens=8, even_split=True)
    a = s.add("a", list(range(1, 20)), max_tokens=2)
    b = s.add("b", list(range(3, 15)), max_tokens=2)
    s.step()
    assert engine.batches[0] == [(0, 0, 4, []), (1, 0, 4, [])]
    s.run()
    assert a.generated == expected(a.prompt, 2) and b.generated == expected(b.prompt, 2)


def test_admission_is_first_come_first_served_and_waits_for_a_slot():
    engine = StandInEngine(num_pages=64, max_slots=2)
    s = Scheduler(engine, max_batch_tokens=64)
    requests = [s.add(i, [i + 1, i + 2], max_tokens=2 + i) for i in range(4)]
    s.step()
    assert [r.slot for r in requests] == [0, 1, None, None] and len(s.queue) == 2
    s.run()
    assert [r.generated for r in requests] == [expected(r.prompt, 2 + i) for i, r in enumerate(requests)]
    order = [r.rid for r in s.finished]
    assert order.index(0) < order.index(2) and s.stats["admitted"] == 4


def test_end_of_sequence_and_limits():
    engine = StandInEngine(num_pages=64)
    stop = expected([5, 6], 3)[2]
    s = Scheduler(engine, eos_token_ids=[stop], context=16)
    r = s.add("r", [5, 6], max_tokens=10)
    clamped = s.add("c", list(range(1, 13)), max_tokens=100)
    too_long = s.add("t", list(range(1, 17)))
    s.run()
    assert r.generated == expected([5, 6], 3) and r.stopped
    assert len(clamped.generated) == 4 and not clamped.stopped        # 16 - 12 tokens of context left
    assert too_long.error == "prompt exceeds request context" and not too_long.generated


def test_pages_run_out_preempt_recompute_and_finish():
    # 6 pages of 4 tokens: two requests of 10 + 12 tokens cannot both reach their full length
    engine = StandInEngine(num_pages=6)
    s = Scheduler(engine, max_batch_tokens=64)
    a = s.add("a", list(range(1, 9)), max_tokens=6)
    b = s.add("b", list(range(2, 10)), max_tokens=6)
    s.run()
    assert a.generated == expected(a.prompt, 6) and b.generated == expected(b.prompt, 6)
    assert s.stats["preemptions"] >= 1 and a.preemptions + b.preemptions == s.stats["preemptions"]
    restarts = [batch for batch in engine.batches[1:] for (_, start, n, _) in batch if start == 0 and n > 1]
    assert restarts, "a preempted request is recomputed from position 0"
    assert engine.cache.available_pages() == 6 and engine.cache.free_slots() == 4


def test_victim_is_the_request_that_already_produced_a_token_then_holds_most_pages():
    engine = StandInEngine(num_pages=5)
    s = Scheduler(engine, max_batch_tokens=8)
    old = s.add("old", list(range(1, 8)), max_tokens=8)           # 7 tokens: 2 pages, then it decodes
    s.step()
    new = s.add("new", list(range(1, 13)), max_tokens=8)          # 12 tokens, 7 of them fit the next step
    s.step()
    assert len(old.generated) == 2 and new.computed == 7 and engine.cache.available_pages() == 1
    s.step()              # old takes the last page for position 8; new's portion stops at its page's end
    assert engine.batches[-1] == [(0, 8, 1, [0]), (1, 7, 1, [])] and engine.cache.available_pages() == 0
    s.step()              # new needs a page and none is free: the request that already decodes is paused
    assert s.stats["preemptions"] == 1 and old.slot is None and new.slot is not None and new.computed > 8
    s.run()
    assert old.generated == expected(old.prompt, 8) and new.generated == expected(new.prompt, 8)


def test_one_request_larger_than_the_pool_is_an_error():
    engine = StandInEngine(num_pages=2)
    s = Scheduler(engine, max_batch_tokens=64)
    s.add("big", list(range(1, 8)), max_tokens=5)
    with pytest.raises(SchedulerError, match="one request exceeded its physical KV capacity"):
        s.run()


def test_a_portion_is_shortened_at_the_page_that_cannot_be_had():
    engine = StandInEngine(num_pages=3)
    s = Scheduler(engine, max_batch_tokens=64)
    a = s.add("a", list(range(1, 7)), max_tokens=1)               # 6 tokens: 2 pages
    b = s.add("b", list(range(1, 11)), max_tokens=1)              # 10 tokens: would need 3 pages
    s.step()
    assert engine.batches[0] == [(0, 0, 6, [5]), (1, 0, 4, [])]   # b gets the one page that is left
    s.run()
    assert a.generated == expected(a.prompt, 1) and b.generated == expected(b.prompt, 1)


def test_host_sampling_is_used_when_the_rule_needs_it():
    engine = StandInEngine(num_pages=16)
    s = Scheduler(engine)
    r = s.add("r", [1, 2, 3], Sampling(temperature=0.7, top_k=5, top_p=0.9, seed=3), max_tokens=5)
    g = s.add("g", [1, 2, 3], Sampling(temperature=0.7, seed=3, presence_penalty=1.5), max_tokens=5)
    s.run()
    assert len(r.generated) == 5 and len(g.generated) == 5


class CandidateStandIn(StandInEngine):
    """The stand-in with the engine's extraction of a row's best candidates and softmax mass."""

    def select_candidates(self, logits, k, temperatures=None):
        rows = logits.numpy()
        order = np.stack([np.lexsort((-np.arange(VOCAB), -row.astype(np.float64)))[:k] for row in rows])
        values = np.take_along_axis(rows, order, axis=1)
        if temperatures is None:
            return values, order.astype(np.int32)
        mass = [(float(row.max()), float(np.exp((row.astype(np.float64) - float(row.max())) / t).sum()) if t else 0.0)
                for row, t in zip(rows, temperatures)]
        return values, order.astype(np.int32), np.array(mass)


def test_rules_without_top_k_draw_from_candidates_or_fall_back_to_the_row_with_the_same_tokens():
    """Cold requests keep one token (settled by the candidates), warm ones keep most of the vocabulary (the whole
    row is fetched); beside them a greedy one and one with top_k.  The same tokens as without the extraction."""
    rules = [Sampling(temperature=0.2, top_p=0.9, seed=1), Sampling(temperature=0.9, top_p=0.9, seed=2), Sampling(),
             Sampling(temperature=0.9, top_k=7, top_p=0.8, seed=3)]
    results = []
    for engine_type in (StandInEngine, CandidateStandIn):
        engine = engine_type(num_pages=64)
        s = Scheduler(engine, max_batch_tokens=16)
        requests = [s.add(i, [3 + i, 5, 8], rule, max_tokens=9) for i, rule in enumerate(rules)]
        s.run()
        results.append([list(r.generated) for r in requests])
        if engine_type is CandidateStandIn:
            assert s.stats["candidate_steps"] > 0 and s.stats["whole_row_draws"] >= 9
            assert s.stats["whole_row_draws"] <= 9 * 2          # never for the cold, the greedy or the top_k request
    assert results[0] == results[1] and all(len(g) == 9 for g in results[0])


class PipelinedStandIn(StandInEngine):
    """The stand-in with the engine's non-waiting selection: tokens become readable only through
    `tokens()`, and a fed step takes them where the device would, from the last selection."""

    class Pending:
        def __init__(self, tokens):
            self.device_tokens, self.read = tokens, False

        def tokens(self):
            self.read = True
            return list(self.device_tokens)

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.fed_steps = 0

    def select_tokens_start(self, logits, samplings, positions):
        return self.Pending(self.select_tokens(logits, samplings, positions))

    def step(self, entries, feed=None):
        if feed is not None:
            assert not feed.read, "a fed step after its tokens were read gains nothing: it should not happen"
            assert all(len(e.tokens) == 1 for e in entries) and len(entries) <= len(feed.device_tokens)
            entries = [type(e)(e.slot, [feed.device_tokens[i]], e.start, e.want) for i, e in enumerate(entries)]
            self.fed_steps += 1
        return super().step(entries)


@pytest.mark.parametrize("seed", range(12))
def test_pipelined_decoding_gives_every_request_the_same_tokens(seed):
    """Random workloads (prompt lengths, limits, end-of-sequence tokens that do occur, few pages so that
    requests are paused, more requests than slots) through the plain and the pipelined scheduler: the same
    tokens for every request, no page lost, and the pipelined one does feed steps on the device."""
    rng = np.random.default_rng(seed)
    jobs = [([int(t) for t in rng.integers(1, VOCAB, size=int(rng.integers(1, 30)))], int(rng.integers(1, 40)))
            for _ in range(int(rng.integers(3, 9)))]
    eos = [int(t) for t in rng.integers(0, VOCAB, size=2)] if seed % 3 else []
    pages = int(rng.integers(24, 60))
    results = []
    for engine_type, pipeline in ((StandInEngine, False), (PipelinedStandIn, True)):
        engine = engine_type(num_pages=pages, page_size=4, max_slots=3, context=128)
        s = Scheduler(engine, max_batch_tokens=int(8 + seed), eos_token_ids=eos, context=128, pipeline=pipeline)
        assert s.pipeline == pipeline
        requests = [s.add(i, prompt, max_tokens=limit) for i, (prompt, limit) in enumerate(jobs)]
        finished = s.run()
        assert len(finished) == len(jobs) and all(r.done for r in requests)
        assert engine.cache.available_pages() == pages and engine.cache.free_slots() == 3
        engine.cache.check()
        results.append([(list(r.generated), r.stopped) for r in requests])
        if pipeline:
            assert s.stats["pipelined_steps"] == engine.fed_steps
            if any(limit > 4 for _, limit in jobs) and not eos:
                assert engine.fed_steps > 0
    assert results[0] == results[1]
    for (prompt, limit), (generated, stopped) in zip(jobs, results[0]):
        want = expected(prompt, limit)
        if not stopped:
            assert generated == want
        else:
            assert generated == want[:len(generated)] and generated[-1] in eos


def test_a_request_ended_by_its_token_has_one_step_computed_for_nobody():
    engine = PipelinedStandIn(num_pages=32)
    prompt = [3, 4]
    stop = expected(prompt, 3)[2]
    assume_distinct = stop not in expected(prompt, 2)
    s = Scheduler(engine, eos_token_ids=[stop], context=64)
    a = s.add("a", prompt, max_tokens=20)
    b = s.add("b", [5, 6, 7], max_tokens=6)
    s.run()
    if assume_distinct:
        assert a.generated == expected(prompt, 3) and a.stopped
    assert b.generated == expected([5, 6, 7], 6)
    assert engine.cache.available_pages() == 32


def test_live_requests_without_a_row_to_run_raise_instead_of_spinning():
    """src/server/paged/schedule.rs:123-125: a step in which requests are live and none can be scheduled is an
    error, not a loop.  The real cache cannot bring that about (a request that needs a page that is not there is
    preempted or refused before the step is planned), so the request is told that all its tokens are computed
    although none was accepted: live, not done, and nothing to run."""
    engine = StandInEngine(num_pages=8)
    s = Scheduler(engine, max_batch_tokens=8, pipeline=False)
    request = s.add("a", [1, 2, 3, 4, 5, 6, 7, 8, 9], max_tokens=4)
    s.prepare()
    assert request.slot == 0 and s.stats["admitted"] == 1
    assert engine.cache.ensure(request.slot, 0, 9)
    s._advance(request, 9)
    with pytest.raises(SchedulerError, match="made no progress"):
        s.step()


@pytest.mark.parametrize("seed", [0, 1, 2, 3])
@pytest.mark.parametrize("even_split", [False, True])
def test_random_requests_on_a_small_pool_all_finish_with_their_tokens(seed, even_split):
    """Random prompts and limits on a pool that cannot hold them all, so requests wait, are cut, preempted and
    computed again: every request ends with the tokens it would get alone, the cache's invariants hold after every
    step (the stand-in checks them), nothing is held at the end, and the face's mirror of a request says what the
    native core says."""
    rng = np.random.default_rng(seed)
    engine = StandInEngine(num_pages=14, page_size=4, max_slots=3, context=64)
    s = Scheduler(engine, max_batch_tokens=int(rng.integers(3, 12)), even_split=even_split, pipeline=False)
    wanted = {}
    for i in range(9):
        prompt = [int(t) for t in rng.integers(0, VOCAB, size=int(rng.integers(1, 30)))]
        limit = int(rng.integers(1, 12))
        wanted[i] = expected(prompt, limit)
        s.add(i, prompt, max_tokens=limit)
    steps = 0
    while s.has_work():
        s.step()
        steps += 1
        assert steps < 2000
        for request in s.live() + list(s.paused) + list(s.queue):
            state = s.core_state(request)
            assert (state["slot"], state["computed"], state["tokens"], state["generated"], state["preemptions"]) == \
                   (request.slot, request.computed, len(request.tokens), len(request.generated), request.preemptions)
    assert {r.rid: r.generated for r in s.finished} == wanted
    assert engine.cache.free_slots() == 3 and engine.cache.available_pages() == 14
    engine.cache.check()


def test_padding_of_single_token_steps_is_a_function_of_the_counts_alone():
    """Up to eight single tokens run as they are; beyond, a step is brought to a multiple of eight rows while the
    step's buffers have room; a step with a portion among its entries is never padded."""
    from types import SimpleNamespace

    from lia_rs_b200.engine.step import StepRuntime
    runtime = SimpleNamespace(max_batch_tokens=64, PAD_ABOVE=StepRuntime.PAD_ABOVE, PAD_TO=StepRuntime.PAD_TO)
    padding = lambda tokens, entries: StepRuntime.padding_for(runtime, tokens, entries)
    assert [padding(n, n) for n in range(1, 9)] == [0] * 8
    assert [padding(n, n) for n in (9, 11, 16, 17, 57, 63, 64)] == [7, 5, 0, 7, 7, 1, 0]
    assert padding(12, 11) == 0 and padding(40, 2) == 0
    runtime.max_batch_tokens = 20
    assert padding(17, 17) == 0 and padding(15, 15) == 1          # 24 rows would not fit the buffers
