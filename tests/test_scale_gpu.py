"""The engine where the benchmark runs it, against the plain implementation: contexts of thousands of tokens
(context buckets 4,096 and 8,192, 16 to 32 ranges of keys per decoded token), 64 live requests (the products
between 17 and 128 tokens as a decode step), and the whole 2B-class model (40 layers, the family's vocabulary)
under the four ways of cutting, in 32-bit and in bfloat16.

The reference holds itself to whole-model logits against an external 32-bit oracle (tests/minicpm5.rs:8-64),
to more than 8,192 tokens of context (tests/minicpm5_long_context.rs:7-97) and to 64 requests side by side
(tests/minicpm5_batches.rs:7-64)."""
import numpy as np
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="module")
def long_models(tmp_path_factory):
    root = tmp_path_factory.mktemp("long_models")
    return {name: helpers.make_model(str(root / name), name) for name in helpers.LONG_8K}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(helpers.LONG_8K))
def test_long_context_in_portions_then_decoding(long_models, name, dtype):
    """One request is filled in portions of changing size to 4,100 tokens, decodes 20 tokens there beside a short
    request, is filled on to 8,000 tokens and decodes 40 more.  Every portion's last row and every decoded row is
    compared with the whole sequence in the plain implementation."""
    from lia_rs_b200.engine import Engine
    model = long_models[name]
    vocab = model["config"]["vocab_size"]
    tokens = helpers.random_tokens(vocab, 8040, 31)
    short = helpers.random_tokens(vocab, 70, 32)
    engine = Engine(model["dir"], dtype=dtype, page_size=model["page_size"], max_tokens=8192 + 128, max_seqs=2,
                    max_batch_tokens=1024)
    replay = helpers.Replayer(engine)
    rows, where = [], []              # logits of the long request and their positions
    rows_short = []

    def fill(upto, sizes):
        at, k = replay.live["long"][1] if "long" in replay.live else 0, 0
        while at < upto:
            n = min(sizes[k % len(sizes)], upto - at)
            k += 1
            rows.append(replay.step([("long", tokens[at:at + n], [n - 1])]))
            where.append(at + n - 1)
            at += n

    fill(4100, [1000, 37, 1024, 512, 2, 900])
    replay.step([("short", short[:10], [])])
    for i in range(20):
        both = replay.step([("long", [tokens[4100 + i]], [0]), ("short", [short[10 + i]], [0])])
        rows.append(both[0:1]); where.append(4100 + i)
        rows_short.append(both[1:2])
    fill(8000, [1024, 1024, 333, 1019])
    for i in range(40):
        both = replay.step([("short", [short[30 + i]], [0]), ("long", [tokens[8000 + i]], [0])])
        rows.append(both[1:2]); where.append(8000 + i)
        rows_short.append(both[0:1])
    buckets = {key[2] for key in engine._graphs} if engine.cuda_graphs else set()
    assert not engine.cuda_graphs or {4096, 8192} <= buckets
    reference = helpers.plain_logits(model, tokens, dtype)
    helpers.assert_close(np.concatenate(rows), reference[where], dtype, f"{name} long request")
    helpers.assert_close(np.concatenate(rows_short), helpers.plain_logits(model, short, dtype)[10:70], dtype,
                         f"{name} short request beside it")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["tiny-D", "tiny-E"])
def test_64_live_requests(tiny_models, name, dtype):
    """64 requests with contexts of 3 to 500 tokens: 8 decode steps of all of them (a product of 64 tokens in every
    layer), then one mixed step of 48 single tokens beside two prompt portions."""
    from lia_rs_b200.engine import Engine
    model = tiny_models[name]
    vocab = model["config"]["vocab_size"]
    lengths = [3 + (97 * i) % 490 for i in range(64)]
    requests = [helpers.random_tokens(vocab, n + 9, 500 + i) for i, n in enumerate(lengths)]
    late = [helpers.random_tokens(vocab, 150, 700), helpers.random_tokens(vocab, 61, 701)]
    engine = Engine(model["dir"], dtype=dtype, page_size=model["page_size"], max_tokens=64 * 512, max_seqs=64,
                    max_batch_tokens=2048)
    replay = helpers.Replayer(engine)
    batch, count = [], 0
    for i, (tokens, n) in enumerate(zip(requests, lengths)):       # prompts, several to a step
        if count + n > 2048:
            replay.step(batch)
            batch, count = [], 0
        batch.append((f"r{i}", tokens[:n], []))
        count += n
    replay.step(batch)
    got = [[] for _ in requests]
    for k in range(8):
        out = replay.step([(f"r{i}", [tokens[n + k]], [0]) for i, (tokens, n) in enumerate(zip(requests, lengths))])
        for i in range(64):
            got[i].append(out[i:i + 1])
    # 16 requests end; two new ones bring portions of their prompts beside the 48 that decode on
    entries = [(f"r{i}", [requests[i][lengths[i] + 8]], [0]) for i in range(48)]
    entries += [("late0", late[0][:100], [99]), ("late1", late[1], [0, 60])]
    for i in range(48, 64):
        replay.engine.release(replay.live.pop(f"r{i}")[0])
    out = replay.step(entries)
    for i in range(48):
        got[i].append(out[i:i + 1])
    for i, (tokens, n) in enumerate(zip(requests, lengths)):
        reference = helpers.plain_logits(model, tokens, dtype)
        steps = 9 if i < 48 else 8
        helpers.assert_close(np.concatenate(got[i]), reference[n:n + steps], dtype, f"{name} request {i} of 64")
    helpers.assert_close(out[48:49], helpers.plain_logits(model, late[0][:100], dtype)[[99]], dtype, f"{name} late portion")
    helpers.assert_close(out[49:51], helpers.plain_logits(model, late[1], dtype)[[0, 60]], dtype, f"{name} late prompt")


@pytest.fixture(scope="module")
def whole_model(tmp_path_factory):
    return helpers.make_model(str(tmp_path_factory.mktemp("whole") / "whole-2B"), "whole-2B")


@pytest.mark.parametrize("dtype", DTYPES)
def test_whole_2b_class_model_under_the_four_ways_of_cutting(whole_model, dtype):
    """All 40 layers and the 73,448-token vocabulary, a 64-token and a 33-token request: each whole; most of one
    in a step and its last 32 tokens one by one; portions of changing size; both mixed in a pool so small that
    pages are used again.  32-bit: against the plain implementation, within the bound of the arithmetic.
    bfloat16: no farther from the exact model than the plain implementation that rounds where the serving path
    does (`helpers.assert_as_accurate_as_rounding` says why element-wise agreement ends at this depth).
    (The plain implementation takes the 2 G parameters through 64-bit products on the CPU: this is the slowest
    test of the suite.)"""
    from lia_rs_b200.engine import Engine
    model = whole_model
    vocab = model["config"]["vocab_size"]
    a, b = helpers.random_tokens(vocab, 64, 41), helpers.random_tokens(vocab, 33, 42)
    exact = {"a": helpers.plain_logits(model, a, "float32"), "b": helpers.plain_logits(model, b, "float32")}
    rounded = {"a": helpers.plain_logits(model, a, dtype), "b": helpers.plain_logits(model, b, dtype)}
    k = helpers.longest_sum(model["config"])

    def check(logits, request, rows, what):
        rows = list(rows)
        if dtype == "float32":
            helpers.assert_close(logits, exact[request][rows], dtype, what, k)
        else:
            helpers.assert_as_accurate_as_rounding(logits, exact[request][rows], rounded[request][rows], what)

    engine = Engine(model["dir"], dtype=dtype, page_size=16, max_tokens=128, max_seqs=4, max_batch_tokens=128)
    replay = helpers.Replayer(engine)
    # whole
    check(replay.step([("a", a, range(64))], end=["a"]), "a", range(64), "2B whole, 64 tokens")
    check(replay.step([("b", b, range(33))], end=["b"]), "b", range(33), "2B whole, 33 tokens")
    # most in one step, the last 32 one by one
    rows = [replay.step([("a", a[:32], [31])])]
    for i in range(32, 64):
        rows.append(replay.step([("a", [a[i]], [0])], end=["a"] if i == 63 else []))
    check(np.concatenate(rows), "a", range(31, 64), "2B last 32 one by one")
    # portions of changing size
    rows, at = [], 0
    for n in [5, 2, 7, 3, 2, 11, 4, 2, 9, 6, 13]:
        n = min(n, 64 - at)
        rows.append(replay.step([("a", a[at:at + n], range(n))], end=["a"] if at + n == 64 else []))
        at += n
    assert at == 64
    check(np.concatenate(rows), "a", range(64), "2B portions")
    # mixed: b decodes while a is filled; the pool (128 tokens) held a before and holds both now
    got_a, got_b = [], []
    got_b.append(replay.step([("b", b[:20], range(20))]))
    both = replay.step([("a", a[:30], range(30)), ("b", [b[20]], [0])])
    got_a.append(both[:30]); got_b.append(both[30:])
    both = replay.step([("b", [b[21]], [0]), ("a", a[30:57], range(27))])
    got_b.append(both[:1]); got_a.append(both[1:])
    for i in range(7):
        both = replay.step([("a", [a[57 + i]], [0]), ("b", [b[22 + i]], [0])])
        got_a.append(both[:1]); got_b.append(both[1:])
    got_b.append(replay.step([("b", b[29:], range(4))], end=["a", "b"]))
    check(np.concatenate(got_a), "a", range(64), "2B mixed, first request")
    check(np.concatenate(got_b), "b", range(33), "2B mixed, second request")
    for group in engine.cache.groups:
        assert group.pool.in_use() == 0
    del engine
    torch.cuda.empty_cache()
