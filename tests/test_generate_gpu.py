"""Generation through the Python entry point and the command line."""
import os
import subprocess
import sys

import pytest

import helpers
import plain_impl

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", list(helpers.TINY))
def test_greedy_generation_float32_equals_the_plain_implementation(tiny_models, name):
    from lia_rs_b200 import generate
    model = tiny_models[name]
    vocab = model["config"]["vocab_size"]
    prompts = [helpers.random_tokens(vocab, n, 40 + n) for n in (1, 7, 16, 33)]
    got = generate(model["dir"], prompts, max_tokens=8, dtype="float32", page_size=model["page_size"],
                   kv_pool_tokens=256, max_sequences=4, prefill_batch=16)
    want = [plain_impl.greedy(model["config"], model["weights"], p, 8) for p in prompts]
    assert got == want


@pytest.mark.parametrize("name", list(helpers.TINY))
def test_greedy_generation_bfloat16_picks_a_maximum_of_the_plain_logits(tiny_models, name):
    from lia_rs_b200 import generate
    model = tiny_models[name]
    vocab = model["config"]["vocab_size"]
    prompts = [helpers.random_tokens(vocab, n, 60 + n) for n in (2, 19, 64)]
    got = generate(model["dir"], prompts, max_tokens=12, dtype="bfloat16", page_size=model["page_size"],
                   kv_pool_tokens=128, max_sequences=2, prefill_batch=24)
    for prompt, tokens in zip(prompts, got):
        assert len(tokens) == 12
        sequence = list(prompt) + tokens
        logits = helpers.plain_logits(model, sequence, "bfloat16")
        for i, token in enumerate(tokens):
            row = logits[len(prompt) - 1 + i]
            assert float(row.max() - row[token]) <= 2 * helpers.tolerance("bfloat16", row), (i, token)


def test_temperature_sampling_is_seeded_and_independent_of_batching(tiny_models):
    from lia_rs_b200.engine.generate import Generator
    model = tiny_models["tiny-B"]
    prompts = [helpers.random_tokens(384, n, 80 + n) for n in (2, 19, 64)]
    g = Generator(model["dir"], dtype="float32", page_size=16, kv_pool_tokens=512, max_sequences=4, prefill_batch=128)
    a = g.generate(prompts, max_tokens=12, temperature=0.8, seed=3)
    b = g.generate(prompts, max_tokens=12, temperature=0.8, seed=3)
    c = g.generate(prompts, max_tokens=12, temperature=0.8, seed=4)
    assert a == b and a != c
    # the host rule in 64-bit on the engine's own logits, replayed by the plain sampler
    for prompt, tokens in zip(prompts, a):
        rng, sequence = plain_impl.MT19937(3), list(prompt)
        for token in tokens:
            row = helpers.plain_logits(model, sequence, "float32")[-1]
            entries = plain_impl.distribution(row.float().tolist(), 0.8, 0, 1.0)
            assert plain_impl.draw(entries, rng) == token
            sequence.append(token)
    # with top_k the device hands over only the best candidates of a row: the same draws as from the whole row
    kept = g.generate(prompts, max_tokens=12, temperature=1.3, top_k=5, top_p=0.9, seed=6)
    assert g.last_scheduler.stats["candidate_steps"] > 0
    for prompt, tokens in zip(prompts, kept):
        rng, sequence = plain_impl.MT19937(6), list(prompt)
        for token in tokens:
            row = helpers.plain_logits(model, sequence, "float32")[-1]
            assert plain_impl.draw(plain_impl.distribution(row.float().tolist(), 1.3, 5, 0.9), rng) == token
            sequence.append(token)
    # without top_k the candidates come with the row's whole softmax mass: cold draws are settled by them, warm ones
    # fetch the row; both give the draws of the whole row
    for temperature, seed in ((0.02, 8), (1.0, 9)):
        kept = g.generate(prompts, max_tokens=12, temperature=temperature, top_p=0.9, seed=seed)
        stats = g.last_scheduler.stats
        assert stats["candidate_steps"] > 0
        # 36 draws: cold ones are settled by the candidates, the warm ones mostly come from whole rows
        assert stats["whole_row_draws"] < 36 if temperature < 1.0 else stats["whole_row_draws"] > 18
        for prompt, tokens in zip(prompts, kept):
            rng, sequence = plain_impl.MT19937(seed), list(prompt)
            for token in tokens:
                row = helpers.plain_logits(model, sequence, "float32")[-1]
                assert plain_impl.draw(plain_impl.distribution(row.float().tolist(), temperature, 0, 0.9), rng) == token
                sequence.append(token)
    # position-keyed Gumbel noise on the device: the same draws alone, together, and in small portions
    together = g.generate(prompts, max_tokens=12, temperature=0.8, seed=5, sampler="murmur3_gumbel")
    alone = [g.generate([p], max_tokens=12, temperature=0.8, seed=5, sampler="murmur3_gumbel")[0] for p in prompts]
    small = Generator(model["dir"], dtype="float32", page_size=16, kv_pool_tokens=512, max_sequences=2, prefill_batch=7)
    assert together == alone == small.generate(prompts, max_tokens=12, temperature=0.8, seed=5, sampler="murmur3_gumbel")


def test_scheduler_under_page_pressure_on_the_device(tiny_models):
    from lia_rs_b200.engine.generate import Generator
    model = tiny_models["tiny-A"]
    prompts = [helpers.random_tokens(256, n, 90 + n) for n in (30, 25, 28, 12)]
    roomy = Generator(model["dir"], dtype="float32", page_size=8, kv_pool_tokens=512, max_sequences=4, prefill_batch=32)
    tight = Generator(model["dir"], dtype="float32", page_size=8, kv_pool_tokens=96, max_sequences=4, prefill_batch=32)
    want = roomy.generate(prompts, max_tokens=20)
    got = tight.generate(prompts, max_tokens=20)
    assert tight.last_scheduler.stats["preemptions"] > 0 and roomy.last_scheduler.stats["preemptions"] == 0
    assert got == want
    tight.engine.cache.check()
    assert tight.engine.cache.available_pages() == 12 and tight.engine.cache.free_slots() == 4


def test_command_line(tiny_models):
    model = tiny_models["tiny-A"]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    prompt = helpers.random_tokens(256, 9, 5)
    ids = ",".join(str(t) for t in prompt)
    run = lambda *args: subprocess.run([sys.executable, os.path.join(root, "bin", "lia"), *args],
                                       capture_output=True, text=True, timeout=600)
    done = run("generate", model["dir"], "128", "--prompt-ids", ids, "--max-tokens", "5", "--dtype", "float32",
               "--page-size", "8", "--kv-pool-tokens", "128", "--max-sequences", "2")
    assert done.returncode == 0, done.stderr[-2000:]
    want = plain_impl.greedy(model["config"], model["weights"], prompt, 5)
    assert done.stdout.strip() == "request=0 tokens=" + ",".join(str(t) for t in want)
    done = run("forward-batch", model["dir"], ids, "--dtype", "float32")
    assert done.returncode == 0, done.stderr[-2000:]
    logits = helpers.plain_logits(model, prompt, "float32")
    lines = done.stdout.strip().splitlines()
    assert len(lines) == 9
    for position, line in enumerate(lines):
        fields = dict(f.split("=") for f in line.split())
        assert int(fields["position"]) == position and int(fields["token"]) == int(logits[position].argmax())
    done = run("forward", model["dir"], ids, "--dtype", "bfloat16")
    assert done.returncode == 0 and done.stdout.count("position=") == 9
