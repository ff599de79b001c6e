"""The engine against the plain implementation, in 32-bit and in bfloat16, under every way of
cutting the work: whole, most + last 32 one by one, portions of changing size, and mixed batches
with so few pages that they are used again."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
MODELS = list(helpers.TINY)
LENGTHS = [1, 2, 9, 17, 41, 70, 100]


def make_engine(model, dtype, max_tokens, max_seqs=4):
    from lia_rs_b200.engine import Engine
    return Engine(model["dir"], dtype=dtype, page_size=model["page_size"], max_tokens=max_tokens,
                  max_seqs=max_seqs, max_batch_tokens=max(256, max_tokens))


def sequences(model, lengths=LENGTHS, seed=11):
    vocab = model["config"]["vocab_size"]
    return {f"r{i}": helpers.random_tokens(vocab, n, seed + i) for i, n in enumerate(lengths)}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", MODELS)
def test_whole(tiny_models, name, dtype):
    model = tiny_models[name]
    engine = make_engine(model, dtype, 128)
    replay = helpers.Replayer(engine)
    for rid, tokens in sequences(model).items():
        logits = replay.step([(rid, tokens, range(len(tokens)))], end=[rid])
        helpers.assert_close(logits, helpers.plain_logits(model, tokens, dtype), dtype, f"{name} {rid} whole")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", MODELS)
def test_prompt_then_last_32_one_by_one(tiny_models, name, dtype):
    model = tiny_models[name]
    engine = make_engine(model, dtype, 128)
    replay = helpers.Replayer(engine)
    for rid, tokens in sequences(model).items():
        if len(tokens) <= 33:
            continue
        reference = helpers.plain_logits(model, tokens, dtype)
        head = len(tokens) - 32
        rows = [replay.step([(rid, tokens[:head], [head - 1])])]
        for i in range(head, len(tokens)):
            rows.append(replay.step([(rid, [tokens[i]], [0])], end=[rid] if i == len(tokens) - 1 else []))
        helpers.assert_close(np.concatenate(rows), reference[head - 1:], dtype, f"{name} {rid} last 32")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", MODELS)
def test_portions_of_changing_size(tiny_models, name, dtype):
    model = tiny_models[name]
    engine = make_engine(model, dtype, 128)
    replay = helpers.Replayer(engine)
    sizes = [5, 2, 7, 3, 2, 11, 4, 2, 9, 6]
    for rid, tokens in sequences(model).items():
        rows, at, k = [], 0, 0
        while at < len(tokens):
            n = min(sizes[k % len(sizes)], len(tokens) - at)
            k += 1
            last = at + n == len(tokens)
            rows.append(replay.step([(rid, tokens[at:at + n], range(n))], end=[rid] if last else []))
            at += n
        helpers.assert_close(np.concatenate(rows), helpers.plain_logits(model, tokens, dtype), dtype,
                             f"{name} {rid} portions")


def mixed_trace(requests, rng, decode_tail=6):
    """Steps of up to four live requests: portions of some beside single tokens of others; a
    request is sometimes left out of a step.  Returns [(entries, end)] with entries
    (id, tokens, want=all)."""
    waiting = list(requests.items())
    live, steps = {}, []
    while waiting or live:
        while waiting and len(live) < 4:
            rid, tokens = waiting.pop(0)
            live[rid] = [tokens, 0]
        entries, end = [], []
        for rid, (tokens, at) in list(live.items()):
            if len(live) > 1 and rng.random() < 0.2:
                continue                                    # left out of this step
            left = len(tokens) - at
            n = 1 if left <= decode_tail else int(min(left - decode_tail, rng.choice([2, 3, 5, 8, 13])))
            entries.append((rid, tokens[at:at + n], range(n)))
            live[rid][1] = at + n
            if at + n == len(tokens):
                end.append(rid)
                del live[rid]
        if entries:
            steps.append((entries, end))
    return steps


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", MODELS)
def test_mixed_batches_with_page_reuse(tiny_models, name, dtype):
    model = tiny_models[name]
    lengths = [33, 7, 64, 19, 1, 50, 16, 41, 2, 27]
    requests = sequences(model, lengths, seed=23)
    ps = model["page_size"]
    # the pool holds the four longest requests at once, far fewer pages than all requests together
    pool_tokens = sum(sorted((n + ps - 1) // ps * ps for n in lengths)[-4:])
    assert sum((n + ps - 1) // ps for n in lengths) > pool_tokens // ps, "pages would not be used again"
    engine = make_engine(model, dtype, pool_tokens)
    replay = helpers.Replayer(engine)
    got = {rid: [] for rid in requests}
    for entries, end in mixed_trace(requests, np.random.default_rng(5)):
        logits = replay.step(entries, end)
        at = 0
        for rid, tokens, want in entries:
            got[rid].append(logits[at:at + len(want)])
            at += len(want)
    for group in engine.cache.groups:
        assert group.pool.in_use() == 0
    for rid, tokens in requests.items():
        helpers.assert_close(np.concatenate(got[rid]), helpers.plain_logits(model, tokens, dtype), dtype,
                             f"{name} {rid} mixed")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", MODELS)
def test_long_decoding(tiny_models, name, dtype):
    model = tiny_models[name]
    total = 200
    tokens = helpers.random_tokens(model["config"]["vocab_size"], total, 77)
    engine = make_engine(model, dtype, 256)
    replay = helpers.Replayer(engine)
    rows = [replay.step([("x", tokens[:3], range(3))])]
    for i in range(3, total):
        rows.append(replay.step([("x", [tokens[i]], [0])]))
    helpers.assert_close(np.concatenate(rows), helpers.plain_logits(model, tokens, dtype), dtype, f"{name} long decode")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(helpers.LONG))
def test_decoding_across_the_end_of_a_context_bucket(tmp_path, name, dtype):
    """A long request decodes from position 1,010 to 1,050 beside a short one: the captured decode step of the
    first bucket of context lengths gives way to the next one's (more ranges of keys per token) at 1,024, and
    the short request's rows ride along through the change."""
    model = helpers.make_model(str(tmp_path / name), name)
    vocab = model["config"]["vocab_size"]
    long_one, short_one = helpers.random_tokens(vocab, 1050, 5), helpers.random_tokens(vocab, 60, 6)
    from lia_rs_b200.engine import Engine
    engine = Engine(model["dir"], dtype=dtype, page_size=model["page_size"], max_tokens=1280, max_seqs=2,
                    max_batch_tokens=512)
    replay = helpers.Replayer(engine)
    replay.step([("long", long_one[:500], [])])
    replay.step([("long", long_one[500:1010], []), ("short", short_one[:2], [])])
    rows_long, rows_short = [], []
    for i in range(40):
        both = replay.step([("short", [short_one[2 + i]], [0]), ("long", [long_one[1010 + i]], [0])])
        rows_short.append(both[0:1])
        rows_long.append(both[1:2])
    decode_shapes = {key[:3] for key in engine._graphs if key[3:5] == (2, 0)}      # two single tokens, no portion
    assert decode_shapes == {(2, 2, 1024), (2, 2, 2048)} and engine.stats["graph_replays"] >= 36
    helpers.assert_close(np.concatenate(rows_long), helpers.plain_logits(model, long_one, dtype)[1010:], dtype,
                         f"{name} across the bucket, long request")
    helpers.assert_close(np.concatenate(rows_short), helpers.plain_logits(model, short_one[:42], dtype)[2:], dtype,
                         f"{name} across the bucket, short request")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", MODELS)
def test_one_captured_step_serves_other_divisions_of_its_tokens(tiny_models, name, dtype):
    """Three steps of 128 tokens in two portions each, divided 70 + 58, 90 + 38 and 60 + 68 at different places of
    their requests: wherever the attention cuts all three into the same number of tiles, they are one shape to the
    engine (the first is launched, the second captured, the third replayed), and every wanted row agrees with the
    plain implementation: where a portion begins and how long it is, the kernels read on the device."""
    model = tiny_models[name]
    vocab = model["config"]["vocab_size"]
    a, b = helpers.random_tokens(vocab, 220, 21), helpers.random_tokens(vocab, 164, 22)
    engine = make_engine(model, dtype, 512)
    replay = helpers.Replayer(engine)
    cuts_a, cuts_b = [0, 70, 160, 220], [0, 58, 96, 164]
    rows = [replay.step([("a", a[cuts_a[i]:cuts_a[i + 1]], [cuts_a[i + 1] - cuts_a[i] - 1]),
                         ("b", b[cuts_b[i]:cuts_b[i + 1]], [cuts_b[i + 1] - cuts_b[i] - 1])]) for i in range(3)]
    got_a, got_b = np.concatenate([r[0:1] for r in rows]), np.concatenate([r[1:2] for r in rows])
    helpers.assert_close(got_a, helpers.plain_logits(model, a, dtype)[[69, 159, 219]], dtype, f"{name} request a")
    helpers.assert_close(got_b, helpers.plain_logits(model, b, dtype)[[57, 95, 163]], dtype, f"{name} request b")
    if engine.cuda_graphs:
        shapes = {key[:5] for key in engine._graphs}
        assert shapes == {(128, 2, 1024, 0, 2)}
        # (these lengths give the same number of tiles for every tile size the attention kernels use: 8, 10, 16, 21,
        # 32, 64 or 128 tokens)
        assert len(engine._graphs) == 1 and engine.stats["graph_replays"] == 2


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", MODELS)
def test_replayed_steps_give_the_bits_of_launched_steps(tiny_models, name, dtype):
    """The same steps through an engine that captures and replays them and through one that launches every kernel
    itself: steps of two portions, of a single token beside a portion, and of three single tokens, each shape three
    times at moving positions so that it is launched, captured and replayed.  Every logit must be the same to the
    bit: a replayed graph lets a kernel start under its predecessor's tail, and a kernel that then reads what is
    not yet written shows here (the kernels add in fixed orders, so nothing else may differ)."""
    from lia_rs_b200.engine import Engine
    model = tiny_models[name]
    vocab = model["config"]["vocab_size"]
    a, b, c = (helpers.random_tokens(vocab, n, seed) for n, seed in ((140, 31), (80, 32), (100, 33)))
    steps = []
    for i in range(3):                                       # two portions
        steps.append([("a", a[40 * i:40 * i + 40], [39]), ("b", b[24 * i:24 * i + 24], [23])])
    for i in range(3):                                       # a single token beside a portion
        steps.append([("a", [a[120 + i]], [0]), ("c", c[31 * i:31 * i + 31], [30])])
    for i in range(3):                                       # single tokens
        steps.append([("c", [c[93 + i]], [0]), ("a", [a[123 + i]], [0]), ("b", [b[72 + i]], [0])])
    outputs = []
    for graphs in (True, False):
        engine = Engine(model["dir"], dtype=dtype, page_size=model["page_size"], max_tokens=512, max_seqs=4,
                        max_batch_tokens=256, cuda_graphs=graphs)
        replay = helpers.Replayer(engine)
        outputs.append([replay.step(step) for step in steps])
        if graphs and engine.cuda_graphs:
            assert engine.stats["graph_replays"] >= 3
    for k, (replayed, launched) in enumerate(zip(*outputs)):
        assert np.array_equal(replayed, launched), f"{name} {dtype}: step {k} differs by {np.abs(replayed - launched).max()}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["tiny-B", "tiny-C", "tiny-E"])
def test_steps_of_single_tokens_padded_to_a_round_number_of_rows(tiny_models, name, dtype):
    """Eleven requests decode side by side, then nine of them, then all eleven fed on the device: beyond eight
    entries a step of single tokens runs with rows of nobody up to a multiple of eight (11 and 9 share one shape),
    and the logits of the real rows are those of the plain implementation."""
    from lia_rs_b200.engine import StepEntry
    model = tiny_models[name]
    vocab = model["config"]["vocab_size"]
    prompts = [helpers.random_tokens(vocab, 9 + 3 * i, 70 + i) for i in range(11)]
    engine = make_engine(model, dtype, 1024, max_seqs=12)
    assert engine.runtime_step.padding_for(11, 11) == 5 and engine.runtime_step.padding_for(8, 8) == 0
    assert engine.runtime_step.padding_for(11, 10) == 0          # a portion among the entries: no padding
    replay = helpers.Replayer(engine)
    names = [f"r{i}" for i in range(11)]
    replay.step([(n, p[:-4], []) for n, p in zip(names, prompts)])
    at = {n: len(p) - 4 for n, p in zip(names, prompts)}      # r9 and r10 sit out the second step
    for live in (names, names[:9], names):
        batch = [(n, [prompts[names.index(n)][at[n]]], [0]) for n in live]
        logits = replay.step(batch)
        assert logits.shape[0] == len(live)
        for row, n in enumerate(live):
            reference = helpers.plain_logits(model, prompts[names.index(n)], dtype)[at[n]:at[n] + 1]
            helpers.assert_close(logits[row:row + 1], reference, dtype, f"{name} padded step, {len(live)} requests, {n}")
            at[n] += 1
    stats = engine.stats
    assert stats["tokens"] == sum(len(p) - 4 for p in prompts) + 11 + 9 + 11
    if engine.cuda_graphs:
        assert any(key[0] == 16 and key[3] == 16 for key in engine._graphs), "11 and 9 single tokens run as 16 rows"
        assert not any(key[0] in (9, 11) for key in engine._graphs)


@pytest.mark.parametrize("name", MODELS)
def test_random_traces_replay_to_the_bit(tiny_models, name):
    """Random traces (portions of 2..40 tokens beside single tokens, up to four requests) launched, captured,
    replayed and launched without graphs: the same bits."""
    limit = tiny_models[name]["config"]["max_position_embeddings"]
    helpers.assert_random_traces_replay_to_the_bit(tiny_models[name], seeds=(11, 12, 13), longest_portion=40,
                                                   long_first_range=(50, min(150, limit // 2)))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", MODELS)
def test_first_tokens_of_a_sequence(tiny_models, name, dtype):
    model = tiny_models[name]
    tokens = helpers.random_tokens(model["config"]["vocab_size"], 4, 3)
    reference = helpers.plain_logits(model, tokens, dtype)
    engine = make_engine(model, dtype, 64)
    replay = helpers.Replayer(engine)
    one_by_one = np.concatenate([replay.step([("a", [t], [0])]) for t in tokens])
    helpers.assert_close(one_by_one, reference, dtype, f"{name} first tokens one by one")
    whole = replay.step([("b", tokens, range(4))], end=["a", "b"])
    helpers.assert_close(whole, reference, dtype, f"{name} first tokens whole")
    # a step that wants nothing still writes the cache
    nothing = replay.step([("c", tokens[:2], [])])
    assert nothing is not None and nothing.shape == (0, model["config"]["vocab_size"])
    tail = replay.step([("c", tokens[2:], [0, 1])], end=["c"])
    helpers.assert_close(tail, reference[2:], dtype, f"{name} after a step that wanted nothing")


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_run_program(tiny_models, tmp_path, dtype):
    """bin/trace_run as a user runs it: steps on standard input, <step>.f32 files, `done` lines."""
    model = tiny_models["tiny-B"]
    vocab = model["config"]["vocab_size"]
    a, b = helpers.random_tokens(vocab, 21, 1), helpers.random_tokens(vocab, 9, 2)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:10], "want": [0, 9]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[10:12], "want": []},
                                {"id": "b", "tokens": b[:8], "want": [7]}], "end": []},
        {"step": 2, "entries": [{"id": "b", "tokens": b[8:], "want": [0]},
                                {"id": "a", "tokens": a[12:], "want": [8]}], "end": ["a", "b"]},
    ]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    done = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", model["dir"],
                           "--dtype", dtype, "--out", str(tmp_path), "--max-tokens", "128"],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True,
                          text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    assert done.stdout.split() == ["done", "0", "done", "1", "done", "2"]
    ref_a, ref_b = helpers.plain_logits(model, a, dtype), helpers.plain_logits(model, b, dtype)
    read = lambda s: np.fromfile(tmp_path / f"{s}.f32", dtype="<f4").reshape(-1, vocab)
    helpers.assert_close(read(0), ref_a[[0, 9]], dtype, "trace step 0")
    helpers.assert_close(read(1), ref_b[[7]], dtype, "trace step 1")
    helpers.assert_close(read(2), torch.cat([ref_b[[8]], ref_a[[20]]]), dtype, "trace step 2")
    with open(tmp_path / "index.json") as f:
        index = json.load(f)
    assert index["vocab_size"] == vocab
    assert index["rows"] == {"0": [["a", 0], ["a", 9]], "1": [["b", 7]], "2": [["b", 8], ["a", 20]]}


def test_replay_function_more_than_four_live_and_a_page_size_that_does_not_divide_64(tiny_models):
    """`replay(model, steps)`: the trace program as a Python call.  Six requests live at once, pages of 12
    tokens, a pool that the requests' rounded counts just fill, so that the second wave reuses pages."""
    from lia_rs_b200 import replay
    model = tiny_models["tiny-D"]
    vocab = model["config"]["vocab_size"]
    requests = {f"r{i}": helpers.random_tokens(vocab, 20 + 9 * i, 40 + i) for i in range(6)}
    later = {f"s{i}": helpers.random_tokens(vocab, 50 + i, 60 + i) for i in range(6)}
    steps = [{"step": 0, "entries": [{"id": k, "tokens": v[:11], "want": [10]} for k, v in requests.items()], "end": []},
             {"step": 1, "entries": [{"id": k, "tokens": v[11:], "want": [len(v) - 12]} for k, v in requests.items()],
              "end": list(requests)},
             {"step": 2, "entries": [{"id": k, "tokens": v, "want": [0, len(v) - 1]} for k, v in later.items()],
              "end": list(later)}]
    logits, index = replay(model["dir"], steps, dtype="float32", max_tokens=6 * 128, max_live=6, page_size=12)
    assert index[1] == [[k, len(v) - 1] for k, v in requests.items()]
    for row, (k, v) in enumerate(requests.items()):
        reference = helpers.plain_logits(model, v, "float32")
        helpers.assert_close(logits[0][row:row + 1], reference[[10]], "float32", f"replay {k} step 0")
        helpers.assert_close(logits[1][row:row + 1], reference[[len(v) - 1]], "float32", f"replay {k} step 1")
    for row, (k, v) in enumerate(later.items()):
        reference = helpers.plain_logits(model, v, "float32")
        helpers.assert_close(logits[2][2 * row:2 * row + 2], reference[[0, len(v) - 1]], "float32", f"replay {k}")


@pytest.mark.parametrize("name", ["tiny-D", "tiny-E"])
@pytest.mark.parametrize("batch", [1, 3, 8, 11, 16])
def test_decode_batches_with_varied_contexts(tiny_models, name, batch):
    """Decode steps of 1 to 16 requests with contexts from a few tokens to hundreds (several ranges of
    keys per token, the window's edge, pages used in scrambled order) against the plain implementation."""
    from lia_rs_b200.engine import Engine
    model = tiny_models[name]
    vocab = model["config"]["vocab_size"]
    lengths = [3 + (37 * i) % 290 for i in range(batch)]
    prompts = [helpers.random_tokens(vocab, n + 6, 100 + i) for i, n in enumerate(lengths)]
    engine = Engine(model["dir"], dtype="bfloat16", page_size=model["page_size"], max_tokens=16 * 320, max_seqs=16,
                    max_batch_tokens=512)
    replay = helpers.Replayer(engine)
    for i, (tokens, n) in enumerate(zip(prompts, lengths)):
        replay.step([(f"r{i}", tokens[:n], [])])
    rows = []
    for k in range(6):
        rows.append(replay.step([(f"r{i}", [tokens[n + k]], [0]) for i, (tokens, n) in enumerate(zip(prompts, lengths))]))
    result = np.stack(rows)                               # [6, batch, vocab]
    for i, (tokens, n) in enumerate(zip(prompts, lengths)):
        reference = helpers.plain_logits(model, tokens, "bfloat16")[n:n + 6]
        helpers.assert_close(result[:, i], reference, "bfloat16", f"{name} request {i}")


@pytest.mark.parametrize("name", MODELS)
def test_float32_logits_are_bit_identical_under_every_way_of_cutting(tiny_models, name):
    """The 32-bit kernels sum every product's K in ascending order per output element and walk a token's keys in an
    order that depends on its position alone, so a position's logits are the same bits whole, one by one, in
    portions, and mixed with other requests on pages that were used before."""
    model = tiny_models[name]
    vocab = model["config"]["vocab_size"]
    a, b = helpers.random_tokens(vocab, 70, 201), helpers.random_tokens(vocab, 45, 202)
    engine = make_engine(model, "float32", 160)
    replay = helpers.Replayer(engine)
    whole_a = replay.step([("a", a, range(70))], end=["a"])
    whole_b = replay.step([("b", b, range(45))], end=["b"])
    # most in one step, the last 32 one by one
    rows = [replay.step([("a", a[:38], range(38))])]
    rows += [replay.step([("a", [a[i]], [0])], end=["a"] if i == 69 else []) for i in range(38, 70)]
    assert np.array_equal(np.concatenate(rows), whole_a), "prompt + last 32 one by one"
    # portions of changing size
    rows, at, k = [], 0, 0
    sizes = [5, 2, 7, 3, 2, 11, 4, 2, 9, 6]
    while at < 70:
        n = min(sizes[k % len(sizes)], 70 - at)
        k += 1
        rows.append(replay.step([("a", a[at:at + n], range(n))], end=["a"] if at + n == 70 else []))
        at += n
    assert np.array_equal(np.concatenate(rows), whole_a), "portions"
    # mixed: portions of one beside single tokens of the other, in both orders within the batch
    got_a, got_b = [], [replay.step([("b", b[:20], range(20))])]
    both = replay.step([("a", a[:33], range(33)), ("b", [b[20]], [0])])
    got_a.append(both[:33]); got_b.append(both[33:])
    both = replay.step([("b", b[21:30], range(9)), ("a", [a[33]], [0])])
    got_b.append(both[:9]); got_a.append(both[9:])
    both = replay.step([("a", a[34:], range(36)), ("b", b[30:], range(15))], end=["a", "b"])
    got_a.append(both[:36]); got_b.append(both[36:])
    assert np.array_equal(np.concatenate(got_a), whole_a), "mixed, first request"
    assert np.array_equal(np.concatenate(got_b), whole_b), "mixed, second request"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["tiny-A", "tiny-C", "tiny-E"])
def test_last_layer_runs_only_the_wanted_rows(tiny_models, name, dtype):
    """A step that wants fewer rows than it brings runs the last layer's output projection, second norm and
    feed-forward for the wanted rows alone (the reference prunes the same way, src/inference/llama_fusion.rs:45-60):
    the logits do not change, the cache is written for every token, and the products shrink."""
    from lia_rs_b200.engine import Engine
    model = tiny_models[name]
    cfg = model["config"]
    tokens = helpers.random_tokens(cfg["vocab_size"], 60, 211)
    reference = helpers.plain_logits(model, tokens, dtype)
    engine = Engine(model["dir"], dtype=dtype, page_size=model["page_size"], max_tokens=256, max_seqs=4,
                    max_batch_tokens=128, profile=True)
    replay = helpers.Replayer(engine)
    # rows {0, last} of one request and no row of another, in one step
    other = helpers.random_tokens(cfg["vocab_size"], 17, 212)
    logits = replay.step([("a", tokens[:40], [0, 39]), ("b", other[:9], [])])
    helpers.assert_close(logits, reference[[0, 39]], dtype, f"{name} rows 0 and last")
    summary = engine.profile_summary()
    layers, hidden, inter = cfg["num_hidden_layers"], cfg["hidden_size"], cfg["intermediate_size"]
    down = sum(v["flops"] for k, v in summary.items() if k.endswith(":down"))
    assert down == 2 * hidden * inter * ((layers - 1) * 49 + 2), "the last layer's down product ran more than two rows"
    out = sum(v["flops"] for k, v in summary.items() if k.endswith(":o"))
    width = cfg["num_attention_heads"] * cfg["head_dim"]
    assert out == 2 * hidden * width * ((layers - 1) * 49 + 2)
    # a step that wants nothing: the last layer only appends to the cache
    nothing = replay.step([("a", tokens[40:50], []), ("b", other[9:], [])])
    assert nothing.shape == (0, cfg["vocab_size"])
    summary = engine.profile_summary()
    assert sum(v["flops"] for k, v in summary.items() if k.endswith(":down")) == 2 * hidden * inter * (layers - 1) * 18
    assert not any(k.endswith(":head") for k in summary)
    # what those steps wrote is what later rows read
    rest = replay.step([("a", tokens[50:], range(10)), ("b", [other[0]], [])], end=["a"])
    helpers.assert_close(rest, reference[50:], dtype, f"{name} after pruned steps")
    # few wanted rows among many tokens: only they attend in the last layer (a different kernel serves them)
    engine.profile = False
    long_tokens = helpers.random_tokens(cfg["vocab_size"], 100, 213)
    logits = replay.step([("c", long_tokens, [3, 57, 99])], end=["c", "b"])
    helpers.assert_close(logits, helpers.plain_logits(model, long_tokens, dtype)[[3, 57, 99]], dtype, f"{name} three of 100 rows")
