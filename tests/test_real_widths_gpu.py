"""The engine at the widths of the real family sizes (few layers, a small vocabulary), against the plain
implementation, in 32-bit and in bfloat16: a prompt whole, in portions, and its last tokens one by one, two
requests decoding side by side.  The tiny configurations find faults of logic; these find the ones that
only show at rows of kilobytes, 16 heads per group and sums of thousands of terms."""
import numpy as np
import pytest

import helpers

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def real_models(tmp_path_factory):
    root = tmp_path_factory.mktemp("real_widths")
    return {name: helpers.make_model(str(root / name), name) for name in helpers.REAL_WIDTHS}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(helpers.REAL_WIDTHS))
def test_real_widths_whole_portions_and_decode(real_models, name, dtype):
    from lia_rs_b200.engine import Engine
    model = real_models[name]
    vocab = model["config"]["vocab_size"]
    first = helpers.random_tokens(vocab, 75, 21)
    second = helpers.random_tokens(vocab, 41, 22)
    ref_first = helpers.plain_logits(model, first, dtype)
    ref_second = helpers.plain_logits(model, second, dtype)
    engine = Engine(model["dir"], dtype=dtype, page_size=model["page_size"], max_tokens=512, max_seqs=4,
                    max_batch_tokens=256)
    replay = helpers.Replayer(engine)
    # whole
    logits = replay.step([("whole", first, range(len(first)))], end=["whole"])
    helpers.assert_close(logits, ref_first, dtype, f"{name} whole")
    # portions, then the last 12 tokens of both requests one by one, side by side
    rows_a = [replay.step([("a", first[:40], range(40))]), replay.step([("a", first[40:63], range(23))])]
    rows_b = [replay.step([("b", second[:29], range(29))])]
    for k in range(12):
        both = replay.step([("a", [first[63 + k]], [0]), ("b", [second[29 + k]], [0])])
        rows_a.append(both[0:1])
        rows_b.append(both[1:2])
    helpers.assert_close(np.concatenate(rows_a), ref_first, dtype, f"{name} portions and decode, first request")
    helpers.assert_close(np.concatenate(rows_b), ref_second, dtype, f"{name} portions and decode, second request")


@pytest.mark.parametrize("name", list(helpers.REAL_WIDTHS))
def test_real_widths_replayed_steps_give_the_bits_of_launched_steps(real_models, name):
    """bfloat16, the kernels the benchmark runs (tcgen05 products and prompt attention, the cluster and the
    few-token products, decode attention in clusters): steps of two portions (100 tokens after 1,500, whose keys are
    cut into ranges, and 200), of single tokens beside a portion, and of single tokens, each shape three times, through an engine that
    replays captured graphs and through one that launches every kernel itself.  The logits must agree to the bit:
    in a replayed graph a kernel starts under its predecessor's tail, and one that reads what is not yet written
    shows here."""
    from lia_rs_b200.engine import Engine
    model = real_models[name]
    vocab = model["config"]["vocab_size"]
    a, b, c = (helpers.random_tokens(vocab, n, seed) for n, seed in ((2000, 41), (700, 42), (400, 43)))
    steps = [[("a", a[:1000], [])], [("a", a[1000:1500], [])]]      # (then a's short portions have their keys cut into ranges)
    for i in range(3):
        steps.append([("a", a[1500 + 100 * i:1600 + 100 * i], [99]), ("b", b[200 * i:200 * i + 200], [199])])
    for i in range(3):
        steps.append([("a", [a[1800 + i]], [0]), ("b", [b[600 + i]], [0]), ("c", c[120 * i:120 * i + 120], [119])])
    for i in range(3):
        steps.append([("c", [c[360 + i]], [0]), ("a", [a[1803 + i]], [0]), ("b", [b[603 + i]], [0])])
    outputs = []
    for graphs in (True, False):
        engine = Engine(model["dir"], dtype="bfloat16", page_size=model["page_size"], max_tokens=4096, max_seqs=4,
                        max_batch_tokens=1024, cuda_graphs=graphs)
        replay = helpers.Replayer(engine)
        outputs.append([replay.step(step) for step in steps])
        if graphs:
            assert engine.cuda_graphs and engine.stats["graph_replays"] >= 3
        del engine, replay
    for k, (replayed, launched) in enumerate(zip(*outputs)):
        if replayed is None or replayed.size == 0:
            continue
        assert np.array_equal(replayed, launched), f"{name}: step {k} differs by {np.abs(replayed - launched).max()}"


@pytest.mark.parametrize("name", list(helpers.REAL_WIDTHS))
def test_real_widths_random_traces_replay_to_the_bit(real_models, name):
    """Random traces (portions of 2..300 tokens beside single tokens, up to four requests, sometimes after a
    prompt of 600..3,000 tokens) launched, captured, replayed and launched without graphs: the same bits."""
    helpers.assert_random_traces_replay_to_the_bit(real_models[name], seeds=(1, 2, 3), longest_portion=300,
                                                   long_first_range=(600, 3000))


@pytest.mark.parametrize("M", [1, 8, 64])
def test_head_product_at_the_family_vocabulary(M):
    """The output product at the family's vocabulary (73,448 rows, no multiple of any tile) against 64-bit."""
    import math
    import torch
    from lia_rs_b200.parts.linear import STORE, linear
    from lia_rs_b200.parts import Runtime
    torch.manual_seed(M)
    V, H = 73448, 2048
    y = torch.randn(M, H, device="cuda:0").to(torch.bfloat16)
    w = (torch.randn(V, H, device="cuda:0") / math.sqrt(H)).to(torch.bfloat16)
    logits = torch.empty(M, V, device="cuda:0")
    linear(Runtime("cuda:0", torch.bfloat16), STORE, y, w, logits, 0.125)
    exact = 0.125 * (y.double() @ w.double().T)
    assert float((logits.double() - exact).abs().max()) < 2e-5 * max(1.0, float(exact.abs().max())) * math.sqrt(H / 64)
