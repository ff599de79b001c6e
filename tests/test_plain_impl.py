"""The plain implementation checked against itself: each part against an even plainer form."""
import math

import torch

import helpers
import plain_impl


def test_rotary_is_a_rotation_by_position_times_frequency():
    x = torch.randn(5, 2, 8, dtype=torch.float64)
    pos = torch.tensor([0, 1, 2, 10, 300])
    y = plain_impl.rotary(x, pos, 10000.0)
    assert torch.equal(y[0], x[0])                                   # position 0 rotates nothing
    for t in range(5):
        for i in range(4):
            angle = float(pos[t]) / 10000.0 ** (2 * i / 8)
            a, b = x[t, 1, i], x[t, 1, i + 4]
            assert abs(y[t, 1, i] - (a * math.cos(angle) - b * math.sin(angle))) < 1e-12
            assert abs(y[t, 1, i + 4] - (b * math.cos(angle) + a * math.sin(angle))) < 1e-12
    # scores depend on the difference of positions only
    q, k = torch.randn(1, 1, 8, dtype=torch.float64), torch.randn(1, 1, 8, dtype=torch.float64)
    s1 = (plain_impl.rotary(q, torch.tensor([7]), 1e4) * plain_impl.rotary(k, torch.tensor([3]), 1e4)).sum()
    s2 = (plain_impl.rotary(q, torch.tensor([104]), 1e4) * plain_impl.rotary(k, torch.tensor([100]), 1e4)).sum()
    assert abs(s1 - s2) < 1e-9


def test_attention_against_loops_with_groups_and_window():
    torch.manual_seed(0)
    T, nq, nkv, d = 9, 4, 2, 8
    q, k, v = (torch.randn(T, n, d, dtype=torch.float64) for n in (nq, nkv, nkv))
    for window in (None, 3):
        out = plain_impl.attention(q, k, v, window)
        for t in range(T):
            for h in range(nq):
                keys = [j for j in range(t + 1) if window is None or j > t - window]
                s = torch.tensor([float(q[t, h] @ k[j, h // 2]) / math.sqrt(d) for j in keys], dtype=torch.float64)
                p = torch.exp(s - s.max())
                p /= p.sum()
                want = sum(p[n] * v[j, h // 2] for n, j in enumerate(keys))
                assert torch.allclose(out[t, h], want, atol=1e-12)


def test_norm_and_feed_forward_and_causality(tmp_path):
    x = torch.randn(3, 10, dtype=torch.float64)
    w = torch.rand(10, dtype=torch.float64)
    y = plain_impl.rms_norm(x, w, 1e-5)
    assert torch.allclose(y, x / torch.sqrt((x ** 2).mean(-1, keepdim=True) + 1e-5) * w)
    model = helpers.make_model(str(tmp_path / "m"), "tiny-C")
    tokens = helpers.random_tokens(301, 30, 1)
    whole = plain_impl.forward(model["config"], model["weights"], tokens)
    prefix = plain_impl.forward(model["config"], model["weights"], tokens[:17])
    assert torch.allclose(whole[:17], prefix, atol=1e-10)           # later tokens do not change earlier logits
    changed = list(tokens)
    changed[2] = (changed[2] + 1) % 301                             # token 2 is outside the window of 21 at 29
    other = plain_impl.forward(model["config"], model["weights"], changed)
    assert not torch.allclose(other[29], whole[29], atol=1e-6)      # ...but the full-attention layer sees it
    rounded = plain_impl.forward(model["config"], model["weights"], tokens, store=plain_impl.round_to_bfloat16)
    assert 0 < float((rounded - whole).abs().max()) < 0.1


def test_scalars_reduce_to_plain_llama_when_absent(tmp_path):
    model = helpers.make_model(str(tmp_path / "m"), "tiny-B")      # scale_emb 1, scale_depth 1, base = hidden
    cfg = dict(model["config"])
    tokens = helpers.random_tokens(384, 12, 2)
    cfg["scale_depth"] = math.sqrt(cfg["num_hidden_layers"])        # multiplier exactly 1
    with_keys = plain_impl.forward(cfg, model["weights"], tokens)
    for key in ("scale_emb", "dim_model_base", "scale_depth"):
        cfg.pop(key)
    assert torch.allclose(plain_impl.forward(cfg, model["weights"], tokens), with_keys, atol=1e-12)
