"""Host sampling against the reference's own test vectors and closed forms, and against the
plain implementation's sampler."""
import math

import numpy as np
import pytest

import plain_impl
from lia_rs_b200.sampling import MT19937, RequestSampler, Sampling, distribution, gumbel_noise, murmur_hash


def test_mt19937_published_vector_and_reference_doubles():
    # src/sampling/random.rs:55-70
    r = MT19937(5489)
    assert [r.next() for _ in range(10)] == [3499211612, 581869302, 3890346734, 3586334585, 545404204,
                                             4161255391, 3922919429, 949333985, 2715962298, 1323567403]
    r = MT19937(5489)
    for _ in range(9999):
        r.next()
    assert r.next() == 4123659995
    r = MT19937(42)
    assert abs(r.uniform() - 0.796542984287846) < 1e-15 and abs(r.uniform() - 0.18343478789336848) < 1e-15
    p = plain_impl.MT19937(42)
    q = MT19937(42)
    assert [p.uniform() for _ in range(700)] == [q.uniform() for _ in range(700)]


def test_distribution_closed_forms():
    logits = np.array([0.0, math.log(2.0), math.log(4.0), -np.inf], dtype=np.float32)
    entries = distribution(logits, 1.0, 0, 1.0)
    assert [t for t, _ in entries] == [2, 1, 0]
    assert np.allclose([p for _, p in entries], [4 / 7, 2 / 7, 1 / 7], atol=1e-7)
    assert [t for t, _ in distribution(logits, 1.0, 2, 1.0)] == [2, 1]
    assert [t for t, _ in distribution(logits, 1.0, 0, 0.5)] == [2]
    assert [t for t, _ in distribution(logits, 1.0, 0, 0.6)] == [2, 1]
    half = distribution(logits, 2.0, 0, 1.0)                      # temperature 2: weights 2, sqrt 2, 1
    assert np.allclose([p for _, p in half], np.array([2, math.sqrt(2), 1]) / (3 + math.sqrt(2)), atol=1e-7)
    ties = distribution(np.array([1.0, 1.0, 1.0], dtype=np.float32), 1.0, 2, 1.0)
    assert [t for t, _ in ties] == [2, 1]                         # ties: the larger id first
    with pytest.raises(ValueError):
        distribution(np.array([np.nan, 1.0], dtype=np.float32), 1.0, 0, 1.0)


def test_matches_the_plain_sampler_draw_by_draw():
    rng = np.random.default_rng(0)
    for temperature, top_k, top_p in [(0.8, 0, 1.0), (1.3, 20, 0.95), (0.5, 3, 0.7)]:
        ours = RequestSampler(Sampling(temperature=temperature, top_k=top_k, top_p=top_p, seed=99))
        theirs = plain_impl.MT19937(99)
        for _ in range(40):
            logits = rng.normal(size=300).astype(np.float32) * 3
            want = plain_impl.draw(plain_impl.distribution(logits, temperature, top_k, top_p), theirs)
            assert ours.sample(logits, 0) == want


@pytest.mark.parametrize("top_p", [0.3, 0.9, 0.999, 1.0])
@pytest.mark.parametrize("spread", [0.05, 3.0])
def test_a_row_sorted_only_as_far_as_the_kept_prefix_needs_gives_the_plain_distribution(top_p, spread):
    """A long row, flat or peaked, with runs of equal logits that straddle where the partial sorts cut."""
    rng = np.random.default_rng(int(top_p * 1000) + int(spread * 100))
    logits = (rng.normal(size=6000) * spread).astype(np.float32)
    order = np.argsort(-logits)
    logits[order[250:262]] = logits[order[250]]                    # a tie across the 256 best
    logits[order[4090:4100]] = logits[order[4090]]                 # and across the 4,096 best
    logits[rng.integers(0, 6000, 50)] = -np.inf
    want = plain_impl.distribution(logits, 0.9, 0, top_p)
    got = distribution(logits, 0.9, 0, top_p)
    assert [t for t, _ in got] == [t for t, _ in want]
    assert np.allclose([p for _, p in got], [p for _, p in want], rtol=1e-12, atol=0)
    logits[np.isneginf(logits)] = -40.0                            # a row to sample from holds finite logits only
    want = plain_impl.distribution(logits, 0.9, 0, top_p)
    ours, theirs = RequestSampler(Sampling(temperature=0.9, top_p=top_p, seed=5)), plain_impl.MT19937(5)
    for _ in range(20):
        assert ours.sample(logits, 0) == plain_impl.draw(want, theirs)


def test_greedy_keeps_the_last_maximum_and_presence_penalty():
    s = RequestSampler(Sampling())
    assert s.sample(np.array([1, 5, 5, 2], dtype=np.float32), 0) == 2
    p = RequestSampler(Sampling(presence_penalty=2.0))
    row = np.array([0, 3, 2.5, 0], dtype=np.float32)
    assert [p.sample(row, i) for i in range(3)] == [1, 2, 1]     # 1 is penalised to 1.0, then 2 to 0.5


def test_gumbel_draw_depends_on_seed_position_token_only():
    assert murmur_hash(42, 0, 0) == murmur_hash(42, 0, 0) and murmur_hash(42, 0, 0) != murmur_hash(42, 1, 0)
    assert all(math.isfinite(gumbel_noise(w)) for w in (0, 1, 65535, 1 << 16, (1 << 32) - 1, 123456789))
    rng = np.random.default_rng(1)
    logits = rng.normal(size=500).astype(np.float32)
    a = RequestSampler(Sampling(temperature=1.0, seed=5, sampler="murmur3_gumbel"))
    b = RequestSampler(Sampling(temperature=1.0, seed=5, sampler="murmur3_gumbel"))
    b.sample(rng.normal(size=500).astype(np.float32), 3)         # an earlier draw does not matter
    assert a.sample(logits, 17) == b.sample(logits, 17)
    counts = np.zeros(3)
    for position in range(3000):                                  # frequencies follow the softmax
        s = RequestSampler(Sampling(temperature=1.0, seed=11, sampler="murmur3_gumbel"))
        counts[s.sample(np.array([0.0, math.log(2.0), math.log(3.0)], dtype=np.float32), position)] += 1
    assert np.allclose(counts / 3000, [1 / 6, 2 / 6, 3 / 6], atol=0.03)


def test_request_fields_defaults_and_refusals():
    s = Sampling.from_request({}, environ={})
    assert (s.temperature, s.top_k, s.top_p, s.seed, s.presence_penalty) == (1.0, 20, 0.95, 42, 0.0)
    assert Sampling.from_request({"temperature": 0}, environ={}).greedy
    assert Sampling.from_request({}, environ={}, top_k_when_absent=0).top_k == 0
    assert Sampling.from_request({"top_k": 5}, environ={}, top_k_when_absent=0).top_k == 5
    assert Sampling.from_request({}, environ={"LIA_SAMPLER": "murmur3_gumbel"}).sampler == "murmur3_gumbel"
    for bad in ({"frequency_penalty": 0.5}, {"repetition_penalty": 1.1}, {"min_p": 0.1}, {"top_k": 21},
                {"top_p": 0.0}, {"presence_penalty": 3}, {"temperature": -1}):
        with pytest.raises(ValueError):
            Sampling.from_request(bad, environ={})
    with pytest.raises(ValueError, match="LIA_SAMPLER"):
        Sampling.from_request({}, environ={"LIA_SAMPLER": "xorshift"})
    assert Sampling(temperature=0.9, sampler="murmur3_gumbel").on_device and not Sampling(temperature=0.9).on_device


def host_candidates(logits, k):
    """The best k entries of a row in the order the sampling rule sorts by: larger logit, then larger id."""
    logits = np.asarray(logits, dtype=np.float32)
    ids = np.nonzero(~np.isneginf(logits))[0]
    order = np.lexsort((-ids, -logits[ids].astype(np.float64)))
    ids = ids[order][:k]
    out_ids = np.full(k, -1, dtype=np.int32)
    out_values = np.full(k, -np.inf, dtype=np.float32)
    out_ids[:ids.size] = ids
    out_values[:ids.size] = logits[ids]
    return out_ids, out_values


@pytest.mark.parametrize("sampler", ["mt19937", "murmur3_gumbel"])
@pytest.mark.parametrize("top_k,top_p,temperature", [(1, 1.0, 0.7), (5, 0.9, 1.3), (20, 0.95, 0.6), (20, 1.0, 2.0), (3, 0.2, 1.0)])
def test_sampling_from_the_best_candidates_equals_sampling_from_the_row(sampler, top_k, top_p, temperature):
    """A rule that keeps at most top_k tokens needs only the row's best top_k (or more) logits: the same draws,
    token by token, with ties between equal logits and with more candidates than the rule keeps."""
    from lia_rs_b200.sampling import RequestSampler, Sampling
    rng = np.random.default_rng(top_k * 7 + int(top_p * 10))
    params = Sampling(temperature=temperature, top_k=top_k, top_p=top_p, seed=11, sampler=sampler)
    whole, few = RequestSampler(params), RequestSampler(params)
    for position in range(40):
        logits = rng.normal(size=300).astype(np.float32)
        logits[rng.integers(0, 300, size=6)] = logits.max()              # ties at the top
        ids, values = host_candidates(logits, max(top_k, int(rng.integers(top_k, 33))))
        assert few.sample_candidates(ids, values, position) == whole.sample(logits, position)
    greedy_whole, greedy_few = RequestSampler(Sampling()), RequestSampler(Sampling())
    logits = rng.normal(size=50).astype(np.float32)
    logits[[7, 31]] = logits.max() + 1.0
    ids, values = host_candidates(logits, 4)
    assert greedy_few.sample_candidates(ids, values, 0) == greedy_whole.sample(logits, 0) == 31
    with pytest.raises(ValueError):
        RequestSampler(Sampling(temperature=1.0, top_k=5, presence_penalty=0.5)).sample_candidates(ids, values, 0)
    with pytest.raises(ValueError):
        RequestSampler(Sampling(temperature=1.0, top_k=20)).sample_candidates(ids, values, 0)      # 4 candidates do not cover 20


def test_a_rule_without_top_k_draws_from_the_candidates_when_they_hold_what_it_keeps():
    """Candidates plus the row's whole softmax mass (summed elsewhere, in another order) give the draws of the whole
    row, or None (and use no random number) when they cannot: a kept prefix longer than the candidates, top_p = 1,
    a cut that lies on top_p * total."""
    from lia_rs_b200.sampling import RequestSampler, Sampling
    from lia_rs_b200.sampling.sampler import nucleus_of_candidates
    rng = np.random.default_rng(3)
    params = Sampling(temperature=0.7, top_k=0, top_p=0.9, seed=21)
    whole, few = RequestSampler(params), RequestSampler(params)
    settled = unsettled = 0
    for position in range(60):
        spread = 8.0 if position % 3 else 0.5                       # peaked rows, and flat ones that keep hundreds
        logits = (rng.normal(size=3000) * spread).astype(np.float32)
        logits[rng.integers(0, 3000, 5)] = logits.max()             # equal logits at the top
        ids, values = host_candidates(logits, 32)
        shifted = (logits.astype(np.float64)[::-1] - float(logits.max())) / 0.7
        mass = (float(logits.max()), math.fsum(np.exp(shifted).tolist()))
        token = few.sample_candidates(ids, values, position, mass)
        if token is None:
            unsettled += 1
            token = few.sample(logits, position)
        else:
            settled += 1
        assert token == whole.sample(logits, position)
    assert settled >= 20 and unsettled >= 10
    two = np.array([0, 1], dtype=np.int32), np.array([0.0, 0.0], dtype=np.float32)
    assert nucleus_of_candidates(*two, 0.0, 2.0, 1.0, 0.5) is None                 # the first token's mass IS top_p * total
    assert [int(t) for t in nucleus_of_candidates(*two, 0.0, 2.0, 1.0, 0.4)[0]] == [0]
    assert [int(t) for t in nucleus_of_candidates(*two, 0.0, 2.0, 1.0, 0.6)[0]] == [0, 1]
    assert nucleus_of_candidates(*two, 0.0, 2.0, 1.0, 1.0) is None
    assert nucleus_of_candidates(*two, 0.0, 40.0, 1.0, 0.5) is None                # most of the mass lies outside
    with pytest.raises(ValueError):
        nucleus_of_candidates(*two, 0.0, float("nan"), 1.0, 0.5)
    with pytest.raises(ValueError):
        RequestSampler(params).sample_candidates(*two, 0)                          # no mass given
