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
