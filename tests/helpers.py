"""Shared by the tests: the tiny configurations, model folders with random weights, traces and
the comparison with the plain implementation."""
from __future__ import annotations

import json
import os

import numpy as np
import torch

import plain_impl

# Tiny configurations of the architecture that differ in every size and option: head counts and
# groups (2:1, multi-query 3:1, 2:1 with a head size that is no power of two), widths, layers,
# vocabulary, theta, eps, tied or untied head, MiniCPM's scalars present or absent, page size, and
# (tiny-C, tiny-E) a sliding window on one of two layers, which gives the cache two groups of pages.
# tiny-D and tiny-E have the head sizes (64, 128) that the persistent decode kernel is built for, so
# their decode steps run through it; the others decode part by part.
TINY = {
    "tiny-A": dict(
        config=dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=64,
                    intermediate_size=192, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                    head_dim=16, vocab_size=256, max_position_embeddings=256, rms_norm_eps=1e-5,
                    rope_theta=10000.0, tie_word_embeddings=True, scale_emb=12, scale_depth=1.4,
                    dim_model_base=32, initializer_range=0.02, hidden_act="silu", torch_dtype="bfloat16"),
        seed=0, page_size=8, sharpen=8.0),
    "tiny-B": dict(
        config=dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=96,
                    intermediate_size=256, num_hidden_layers=3, num_attention_heads=3, num_key_value_heads=1,
                    head_dim=32, vocab_size=384, max_position_embeddings=512, rms_norm_eps=1e-6,
                    rope_theta=1e6, tie_word_embeddings=False, scale_emb=1, scale_depth=1.0,
                    dim_model_base=96, initializer_range=0.05, hidden_act="silu", torch_dtype="bfloat16"),
        seed=2, page_size=16, sharpen=3.0),
    "tiny-C": dict(
        config=dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=144,
                    intermediate_size=200, num_hidden_layers=2, num_attention_heads=6, num_key_value_heads=3,
                    head_dim=48, vocab_size=301, max_position_embeddings=384, rms_norm_eps=3e-6,
                    rope_theta=50000.0, tie_word_embeddings=False, sliding_window=21,
                    layer_types=["sliding_attention", "full_attention"], initializer_range=0.03,
                    hidden_act="silu", torch_dtype="bfloat16"),
        seed=7, page_size=4, sharpen=5.0),
    "tiny-D": dict(
        config=dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=128,
                    intermediate_size=264, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2,
                    head_dim=64, vocab_size=500, max_position_embeddings=512, rms_norm_eps=1e-5,
                    rope_theta=10000.0, tie_word_embeddings=True, scale_emb=4, scale_depth=1.2,
                    dim_model_base=64, initializer_range=0.04, hidden_act="silu", torch_dtype="bfloat16"),
        seed=5, page_size=16, sharpen=2.0),
    "tiny-E": dict(
        config=dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=192,
                    intermediate_size=328, num_hidden_layers=2, num_attention_heads=6, num_key_value_heads=1,
                    head_dim=128, vocab_size=333, max_position_embeddings=512, rms_norm_eps=2e-6,
                    rope_theta=300000.0, tie_word_embeddings=False, sliding_window=37,
                    layer_types=["full_attention", "sliding_attention"], initializer_range=0.03,
                    hidden_act="silu", torch_dtype="bfloat16"),
        seed=9, page_size=8, sharpen=1.5),
}

# `sharpen`: q and k projections are scaled up so that attention is peaked: with the usual small
# random weights every key gets nearly the same probability and a wrong or missing key would hide.


# Few layers at the widths of the real family sizes (2B-, 0.5B- and 8B-class: hidden, heads, groups, head size,
# intermediate and MiniCPM's scalars as published; a vocabulary cut to a few thousand, no power of two, so
# that the plain implementation on the CPU stays a matter of seconds).  They put the kernels at the sizes the
# benchmark runs: rows of 4 to 32 KB, 16 query heads per kv head, K of 16384.
REAL_WIDTHS = {
    "width-2B": dict(
        config=dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=2048,
                    intermediate_size=6144, num_hidden_layers=2, num_attention_heads=16, num_key_value_heads=2,
                    head_dim=128, vocab_size=7001, max_position_embeddings=4096, rms_norm_eps=1e-5,
                    rope_theta=10000.0, tie_word_embeddings=True, scale_emb=12, scale_depth=1.4,
                    dim_model_base=256, initializer_range=0.02, hidden_act="silu", torch_dtype="bfloat16"),
        seed=0, page_size=16, sharpen=2.0),
    "width-0.5B": dict(
        config=dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=1024,
                    intermediate_size=4096, num_hidden_layers=2, num_attention_heads=16, num_key_value_heads=2,
                    head_dim=64, vocab_size=5003, max_position_embeddings=4096, rms_norm_eps=1e-5,
                    rope_theta=10000.0, tie_word_embeddings=True, scale_emb=12, scale_depth=1.4,
                    dim_model_base=256, initializer_range=0.02, hidden_act="silu", torch_dtype="bfloat16"),
        seed=4, page_size=16, sharpen=2.0),
    "width-8B": dict(
        config=dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=4096,
                    intermediate_size=16384, num_hidden_layers=1, num_attention_heads=32, num_key_value_heads=2,
                    head_dim=128, vocab_size=3001, max_position_embeddings=4096, rms_norm_eps=1e-5,
                    rope_theta=10000.0, tie_word_embeddings=False, scale_emb=12, scale_depth=1.4,
                    dim_model_base=256, initializer_range=0.02, hidden_act="silu", torch_dtype="bfloat16"),
        seed=5, page_size=16, sharpen=2.0),
}


# Two of the tiny configurations with room for more than a thousand positions: decode steps are captured and
# replayed within a bucket of context lengths (the first ends at 1,024), so a request that decodes across that
# length changes the captured step, the number of ranges its keys are cut into, and the merge.
LONG = {
    "long-B": dict(TINY["tiny-B"], config=dict(TINY["tiny-B"]["config"], max_position_embeddings=1280)),
    "long-E": dict(TINY["tiny-E"], config=dict(TINY["tiny-E"]["config"], max_position_embeddings=1280)),
}


# Two of the tiny configurations with room for 8,192 positions (head sizes 64 and 128, the tensor-core attention
# kernels' sizes): prompts filled in portions to thousands of tokens and decoded there, so that the context buckets
# 4,096 and 8,192 and 16 to 32 ranges of keys per decoded token run against the plain implementation.
LONG_8K = {
    "8k-D": dict(TINY["tiny-D"], config=dict(TINY["tiny-D"]["config"], max_position_embeddings=8192)),
    "8k-E": dict(TINY["tiny-E"], config=dict(TINY["tiny-E"]["config"], max_position_embeddings=8192)),
}

# The 2B-class model whole: every layer, the family's vocabulary.
WHOLE = {
    "whole-2B": dict(
        config=dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=2048,
                    intermediate_size=6144, num_hidden_layers=40, num_attention_heads=16, num_key_value_heads=2,
                    head_dim=128, vocab_size=73448, max_position_embeddings=32768, rms_norm_eps=1e-5,
                    rope_theta=10000.0, tie_word_embeddings=True, scale_emb=12, scale_depth=1.4,
                    dim_model_base=256, initializer_range=0.02, hidden_act="silu", torch_dtype="bfloat16"),
        seed=0, page_size=16, sharpen=2.0),
}


def entry_of(name: str) -> dict:
    for table in (TINY, LONG, LONG_8K, REAL_WIDTHS, WHOLE):
        if name in table:
            return table[name]
    raise KeyError(name)


def make_model(folder: str, name: str) -> dict:
    """Write the folder through the package's random-weights mode, then sharpen q/k and rewrite.
    Returns {dir, config (dict), weights (dict by checkpoint name, as stored), page_size}."""
    from safetensors.torch import load_file, save_file

    from lia_rs_b200 import LlamaConfig, write_random_model
    entry = entry_of(name)
    write_random_model(LlamaConfig.from_dict(entry["config"]), folder, seed=entry["seed"])
    path = os.path.join(folder, "model.safetensors")
    weights = load_file(path)            # the safetensors library, independent of the package's reader
    for key in list(weights):
        if key.endswith("q_proj.weight") or key.endswith("k_proj.weight"):
            weights[key] = (weights[key].float() * entry["sharpen"]).to(torch.bfloat16)
    save_file(weights, path)
    with open(os.path.join(folder, "config.json")) as f:
        config = json.load(f)
    return dict(dir=folder, config=config, weights=weights, page_size=entry["page_size"], name=name)


def random_tokens(vocab: int, count: int, seed: int) -> list:
    rng = np.random.default_rng(seed)
    return [int(t) for t in rng.integers(0, vocab, size=count)]


_PLAIN_CACHE = {}


def rounds_probabilities(head_dim: int) -> bool:
    """The bfloat16 path's tensor-core attention kernels (head sizes 32, 64 and 128) feed 16-bit
    probabilities to the tensor cores; the kernel for every other head size keeps them in 32-bit."""
    return head_dim in (32, 64, 128)


def plain_logits(model: dict, tokens, dtype: str = "float32") -> torch.Tensor:
    """64-bit logits [T, V] of the plain implementation (cached per model and sequence): the exact
    model for the 32-bit path; for the bfloat16 path the model with the values that path keeps in
    16 bits rounded at the same places."""
    key = (model["name"], tuple(tokens), dtype)
    _LAST_MODEL["longest_sum"] = longest_sum(model["config"])
    if key not in _PLAIN_CACHE:
        store = plain_impl._identity if dtype == "float32" else plain_impl.round_to_bfloat16
        store_p = None
        if dtype != "float32" and rounds_probabilities(plain_impl.head_dim_of(model["config"])):
            store_p = plain_impl.round_to_bfloat16
        _PLAIN_CACHE[key] = plain_impl.forward(model["config"], model["weights"], tokens, torch.float64,
                                               store=store, store_p=store_p)
    return _PLAIN_CACHE[key]


# Tolerances, fixed once from the size of rounding in each path and never widened to pass:
#  * float32: from the arithmetic.  A sum of K products in 32-bit is off by at most K units of 2^-24 of the
#    sum of the terms' sizes; 4 K 2^-24 times the largest logit leaves room for the layers that such sums
#    pass through.  K is the longest sum of the model (its widest matrix side): `plain_logits` notes it for
#    the model it was last asked about in the running test, which is the model of the comparison that follows.
#    A comparison that names no model (the toy parts of the tests, whose own arithmetic is the library's
#    32-bit operations) takes 1,024.
#  * bfloat16: compared with the plain implementation that rounds to bfloat16 where the serving path
#    stores 16-bit values.  What remains is the order of sums and a value here and there that rounds
#    the other way (one unit of 2^-8 relative in one stored element).
_LAST_MODEL = {"longest_sum": None}


def longest_sum(config: dict) -> int:
    return max(config["hidden_size"], config["intermediate_size"],
               config["num_attention_heads"] * plain_impl.head_dim_of(config))


def tolerance(dtype: str, reference: torch.Tensor, k: int = None) -> float:
    scale = max(1.0, float(reference.abs().max()))
    if dtype == "float32":
        return 4.0 * (k or _LAST_MODEL["longest_sum"] or 1024) * 2.0 ** -24 * scale
    return 1e-2 * scale


def assert_close(actual, reference, dtype: str, what: str, k: int = None):
    actual = torch.as_tensor(np.asarray(actual), dtype=torch.float64)
    reference = reference.to(torch.float64)
    assert actual.shape == reference.shape, f"{what}: shape {tuple(actual.shape)} vs {tuple(reference.shape)}"
    assert torch.isfinite(actual).all(), f"{what}: non-finite logits"
    error = (actual - reference).abs()
    worst = float(error.max())
    limit = tolerance(dtype, reference, k)
    if worst > limit:
        row = int(error.max(dim=-1).values.argmax()) if error.dim() > 1 else 0
        raise AssertionError(f"{what}: max abs error {worst:.3e} > {limit:.3e} (first at wanted row {row})")


def assert_as_accurate_as_rounding(actual, exact, rounded, what: str, margin: float = 1.25):
    """For a deep model in bfloat16.  After tens of layers two computations that round to 16 bits at the same
    places but add in different orders no longer agree element by element: each is the exact model plus rounding
    noise of its own (measured on the 40-layer model: the plain implementation with rounding is off the exact one
    by 4 % of a logit's size, and so is the engine).  So the engine is held to being no farther from the EXACT
    model than the plain implementation with rounding is, in the root mean square and at the worst logit, with a
    quarter of margin; a fault (a wrong key, a missing layer, a wrong scale) is far outside that."""
    actual = torch.as_tensor(np.asarray(actual), dtype=torch.float64)
    exact, rounded = exact.to(torch.float64), rounded.to(torch.float64)
    assert actual.shape == exact.shape == rounded.shape, f"{what}: shapes differ"
    assert torch.isfinite(actual).all(), f"{what}: non-finite logits"
    rms = lambda x: float(x.pow(2).mean().sqrt())
    ours, theirs = actual - exact, rounded - exact
    assert rms(ours) <= margin * rms(theirs), f"{what}: rms error {rms(ours):.3e} > {margin} x {rms(theirs):.3e}"
    worst, allowed = float(ours.abs().max()), margin * float(theirs.abs().max())
    assert worst <= allowed, f"{what}: max abs error {worst:.3e} > {allowed:.3e}"


class Replayer:
    """Drives an Engine the way bin/trace_run does, in process: requests by name, their positions,
    reservation of pages, release at `end`."""

    def __init__(self, engine):
        self.engine = engine
        self.live = {}

    def step(self, entries, end=()):
        from lia_rs_b200.engine import StepEntry
        batch = []
        for name, tokens, want in entries:
            if name not in self.live:
                self.live[name] = [self.engine.admit(), 0]
            slot, fed = self.live[name]
            assert self.engine.reserve(slot, fed, fed + len(tokens)), "pool exhausted"
            batch.append(StepEntry(slot, list(tokens), fed, list(want)))
            self.live[name][1] = fed + len(tokens)
        logits = self.engine.step(batch).float().cpu().numpy().copy() if batch else None
        self.engine.synchronize()
        for name in end:
            self.engine.release(self.live.pop(name)[0])
        self.engine.cache.check()
        return logits


def random_trace(rng, vocab, max_positions, longest_portion, long_first):
    """A random trace for up to four requests: steps of one to four entries, each a portion of 2..longest_portion
    tokens or, for a request that has begun, a single token half of the time; `long_first` > 0 opens with one long
    portion of the first request, so that later short portions see a long context.  Returns (steps, tokens): steps
    of (request, count, wanted places), tokens by request."""
    ids = ["a", "b", "c", "d"]
    fed = {i: 0 for i in ids}
    steps = []
    if long_first:
        steps.append([("a", long_first, [])])
        fed["a"] = long_first
    for _ in range(rng.randint(4, 9)):
        entries = []
        for i in rng.sample(ids, rng.randint(1, 4)):
            count = 1 if (fed[i] > 0 and rng.random() < 0.5) else rng.randint(2, longest_portion)
            if fed[i] + count > max_positions - 2:
                continue
            want = sorted(rng.sample(range(count), min(count, rng.choice([0, 1, 1, 2])))) if count > 1 else [0]
            if count > 1 and rng.random() < 0.7 and (count - 1) not in want:
                want.append(count - 1)
            entries.append((i, count, want))
            fed[i] += count
        if entries:
            steps.append(entries)
    tokens = {i: random_tokens(vocab, max(fed[i], 1), rng.randint(0, 1 << 30)) for i in ids}
    return steps, tokens


def run_trace(engine, steps, tokens):
    """The trace through the engine, every request ended after the last step; the logits of every step."""
    replay = Replayer(engine)
    at = {}
    outputs = []
    for step in steps:
        batch = []
        for request, count, want in step:
            start = at.get(request, 0)
            batch.append((request, tokens[request][start:start + count], want))
            at[request] = start + count
        outputs.append(replay.step(batch))
    replay.step([], end=list(replay.live))
    return outputs


def assert_random_traces_replay_to_the_bit(model, seeds, longest_portion, long_first_range):
    """Random traces, each three times through an engine with graphs (launched, captured, replayed: a pass ends
    every request, so the next one has the same shapes at the same positions, on other pages) and once through an
    engine that launches every kernel: all four must agree to the bit."""
    import random

    from lia_rs_b200.engine import Engine
    vocab = model["config"]["vocab_size"]
    for seed in seeds:
        rng = random.Random(seed)
        low, high = long_first_range
        long_first = rng.choice([0, rng.randint(low, high)])
        steps, tokens = random_trace(rng, vocab, model["config"]["max_position_embeddings"], longest_portion, long_first)
        pool = sum((len(t) + 63) // 64 * 64 for t in tokens.values()) + 64
        widest = max(sum(count for _, count, _ in step) for step in steps)
        outputs = []
        for graphs in (True, False):
            engine = Engine(model["dir"], dtype="bfloat16", page_size=model["page_size"], max_tokens=pool, max_seqs=4,
                            max_batch_tokens=widest, cuda_graphs=graphs)
            for _ in range(3 if graphs else 1):
                outputs.append(run_trace(engine, steps, tokens))
            if graphs and engine.cuda_graphs:
                assert engine.stats["graph_replays"] >= len(steps)
            del engine
        launched = outputs[-1]
        for p, replayed in enumerate(outputs[:-1]):
            for k, (x, y) in enumerate(zip(replayed, launched)):
                if x is None or x.size == 0:
                    continue
                assert np.array_equal(x, y), (f"{model['name']} seed {seed}, pass {p}, step {k} "
                                              f"{[(r, c) for r, c, _ in steps[k]]}: differs by {np.abs(x - y).max()}")
