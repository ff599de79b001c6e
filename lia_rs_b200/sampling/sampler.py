"""Sampling as the reference does it (src/sampling.rs, src/server/sampling.rs).

Request fields and their defaults: `temperature` (0 = greedy), `top_k` (0 = unrestricted, at most
20), `top_p` in (0, 1], `seed` (42), `presence_penalty` in [-2, 2] (0).  frequency_penalty,
repetition_penalty and min_p are rejected unless at their neutral value
(src/server/sampling.rs:65-71).

Greedy keeps the LAST maximal index (src/server/paged/request.rs:117-124).  With a temperature the
distribution is built in 64-bit: sort by descending logit (ties: larger id first), keep top_k,
weights exp((x - max)/T), keep the shortest prefix whose mass reaches top_p * total, renormalise
(src/sampling.rs:82-131).  Two random sources:
  * "mt19937": MT19937 seeded with the low 32 bits of the seed; one 64-bit uniform from two words;
    inverse CDF over the sorted entries; a single entry draws nothing (src/sampling/random.rs:8-46,
    src/sampling.rs:134-186).  The draw depends on how many draws came before.
  * "murmur3_gumbel": Gumbel-max with noise keyed by (seed, position, token), so a draw does not
    depend on batching or on earlier draws (src/sampling/gumbel.rs:4-52).  Without top_k/top_p and
    penalty this runs on the device (csrc/sampling.cu).
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass

import numpy as np

SAMPLERS = ("mt19937", "murmur3_gumbel")


@dataclass(frozen=True)
class Sampling:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    seed: int = 42
    presence_penalty: float = 0.0
    sampler: str = "mt19937"

    def __post_init__(self):
        if not (math.isfinite(self.temperature) and self.temperature >= 0.0):
            raise ValueError("invalid temperature")
        if not 0 <= int(self.top_k) <= 20:
            raise ValueError("sampling top_k must be 0 (unrestricted) or 1..=20")
        if not (math.isfinite(self.top_p) and 0.0 < self.top_p <= 1.0):
            raise ValueError("top_p must be in (0,1]")
        if not (math.isfinite(self.presence_penalty) and -2.0 <= self.presence_penalty <= 2.0):
            raise ValueError("invalid presence_penalty")
        if self.sampler not in SAMPLERS:
            raise ValueError(f"invalid sampler {self.sampler!r}; known: {SAMPLERS}")
        if self.seed < 0:
            raise ValueError("invalid seed")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0

    @property
    def on_device(self) -> bool:
        """Whether the device kernel computes exactly this request's rule."""
        if self.presence_penalty != 0.0:
            return False
        if self.greedy:
            return True
        return self.sampler == "murmur3_gumbel" and self.top_k == 0 and self.top_p == 1.0

    @classmethod
    def from_request(cls, request: dict, environ=None, top_k_when_absent: int = 20) -> "Sampling":
        """Build from a request's JSON fields with the reference's names, defaults and refusals
        (src/server/sampling.rs:32-90).  LIA_DEFAULT_TEMPERATURE, LIA_DEFAULT_PRESENCE_PENALTY and
        LIA_SAMPLER are honoured as there.  A request without top_k gets 20; the paged service of this
        architecture passes `top_k_when_absent=0`, unrestricted (src/server/paged/request.rs:49-52)."""
        environ = os.environ if environ is None else environ

        def number(name, default):
            value = request.get(name)
            if value is None:
                return default
            if isinstance(value, bool) or not isinstance(value, (int, float)):
                raise ValueError(f"invalid {name}")
            return float(value)

        def integer(name, default):
            value = request.get(name)
            if value is None:
                return default
            if isinstance(value, bool) or not isinstance(value, int) or value < 0:
                raise ValueError(f"invalid {name}")
            return value

        for name, neutral in (("frequency_penalty", 0.0), ("repetition_penalty", 1.0), ("min_p", 0.0)):
            if number(name, neutral) != neutral:
                raise ValueError(f"unsupported {name}")
        try:
            default_temperature = float(environ.get("LIA_DEFAULT_TEMPERATURE", 1.0))
            default_presence = float(environ.get("LIA_DEFAULT_PRESENCE_PENALTY", 0.0))
        except ValueError as error:
            raise ValueError(f"invalid LIA_DEFAULT_TEMPERATURE or LIA_DEFAULT_PRESENCE_PENALTY: {error}")
        sampler = environ.get("LIA_SAMPLER", "mt19937")
        if sampler not in SAMPLERS:
            raise ValueError(f"invalid LIA_SAMPLER: {sampler}")
        return cls(temperature=number("temperature", default_temperature), top_k=integer("top_k", top_k_when_absent),
                   top_p=number("top_p", 0.95), seed=integer("seed", 42),
                   presence_penalty=number("presence_penalty", default_presence), sampler=sampler)


class MT19937:
    """The reference's generator (src/sampling/random.rs:8-46), the twist vectorised."""

    def __init__(self, seed: int):
        words = np.zeros(624, dtype=np.uint64)
        words[0] = seed & 0xFFFFFFFF
        for i in range(1, 624):
            prev = int(words[i - 1])
            words[i] = (1812433253 * (prev ^ (prev >> 30)) + i) & 0xFFFFFFFF
        self.words = [int(w) for w in words]
        self.index = 624

    def _twist(self):
        w = self.words
        for i in range(624):
            mixed = (w[i] & 0x80000000) | (w[(i + 1) % 624] & 0x7FFFFFFF)
            w[i] = w[(i + 397) % 624] ^ (mixed >> 1) ^ (0x9908B0DF if mixed & 1 else 0)
        self.index = 0

    def next(self) -> int:
        if self.index == 624:
            self._twist()
        value = self.words[self.index]
        self.index += 1
        value ^= value >> 11
        value ^= (value << 7) & 0x9D2C5680
        value ^= (value << 15) & 0xEFC60000
        return (value ^ (value >> 18)) & 0xFFFFFFFF

    def uniform(self) -> float:
        low, high = float(self.next()), float(self.next())
        return min((low + high * 4294967296.0) / 18446744073709551616.0, math.nextafter(1.0, 0.0))


def _rotl(x: int, r: int) -> int:
    return ((x << r) | (x >> (32 - r))) & 0xFFFFFFFF


def murmur_hash(seed: int, position: int, token: int) -> int:
    h = 0
    for word in (seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF, position & 0xFFFFFFFF, token & 0xFFFFFFFF):
        k = (_rotl((word * 0xCC9E2D51) & 0xFFFFFFFF, 15) * 0x1B873593) & 0xFFFFFFFF
        h = (_rotl(h ^ k, 13) * 5 + 0xE6546B64) & 0xFFFFFFFF
    h ^= 16
    h ^= h >> 16
    h = (h * 0x85EBCA6B) & 0xFFFFFFFF
    h ^= h >> 13
    h = (h * 0xC2B2AE35) & 0xFFFFFFFF
    return h ^ (h >> 16)


def gumbel_noise(word: int) -> float:
    f = np.float32
    u = f(f(word >> 16) * f(1.0 / 65536.0) + f(f(word & 65535) + f(0.5)) * f(1.0 / 4294967296.0))
    if u < f(0.25):
        poly = f(1.0 / 8.0)
        for den in range(7, 0, -1):
            poly = f(u * poly + f(1.0 / den))
        negative_log = f(u * poly)
    else:
        negative_log = f(-np.log(max(f(1.0) - u, f(1.0 / 16777216.0)), dtype=np.float32))
    return float(-np.log(negative_log, dtype=np.float32))


def _best_first(logits: np.ndarray, ids: np.ndarray, at_least: int) -> np.ndarray:
    """A prefix of `ids` in the rule's order (larger logit first, among equal ones the larger id) that holds at
    least the `at_least` best: everything not below the at_least-th largest logit, so no tie is cut."""
    values = logits[ids]
    if at_least < ids.size:
        bound = np.partition(values, ids.size - at_least)[ids.size - at_least]
        chosen = values >= bound
        ids, values = ids[chosen], values[chosen]
    return ids[np.lexsort((-ids, -values.astype(np.float64)))]


def distribution_arrays(logits: np.ndarray, temperature: float, top_k: int, top_p: float):
    """(tokens, probabilities) of the kept entries, best first, as described in the module's header.  Only as
    much of the row is sorted as the kept prefix needs: without top_k the total mass is summed over the row as it
    lies, and the best 256, 4,096, ... entries are sorted until their running mass reaches top_p of it."""
    logits = np.asarray(logits, dtype=np.float32)
    if np.isnan(logits).any() or np.isposinf(logits).any():
        raise ValueError("invalid sampling logits")
    ids = np.nonzero(~np.isneginf(logits))[0]
    if ids.size == 0:
        raise ValueError("empty sampling distribution")
    if top_k:
        best = _best_first(logits, ids, top_k)[:top_k]
        weights = np.exp((logits[best].astype(np.float64) - float(logits[best[0]])) / temperature)
        mass = np.cumsum(weights)
        reach = np.nonzero(mass >= top_p * float(weights.sum()))[0]
    else:
        largest = float(logits[ids].max())
        total = float(np.exp((logits[ids].astype(np.float64) - largest) / temperature).sum())
        sorted_so_far = 256 if top_p < 1.0 else ids.size          # the whole mass is reached at the end only
        while True:
            best = _best_first(logits, ids, sorted_so_far)
            weights = np.exp((logits[best].astype(np.float64) - largest) / temperature)
            mass = np.cumsum(weights)
            reach = np.nonzero(mass >= top_p * total)[0]
            if reach.size or best.size == ids.size:
                break
            # sixteen times as many next time; all of them when that is most of the row, or when the best so far
            # hold so little of the mass that the kept prefix must be long
            sorted_so_far = sorted_so_far * 16 if float(mass[-1]) * 4 >= top_p * total else ids.size
            if sorted_so_far * 4 >= ids.size:
                sorted_so_far = ids.size
    keep = int(reach[0]) + 1 if reach.size else best.size
    weights = weights[:keep]
    return best[:keep], weights / float(weights.sum())


def distribution(logits: np.ndarray, temperature: float, top_k: int, top_p: float) -> list:
    """Sorted [(token, probability)] as described in the module's header."""
    tokens, probabilities = distribution_arrays(logits, temperature, top_k, top_p)
    return list(zip((int(i) for i in tokens), (float(w) for w in probabilities)))


def distribution_of_candidates(ids, values, temperature: float, top_k: int, top_p: float):
    """`distribution_arrays` for a row of which only the best candidates are known: `ids` and `values` hold at least
    top_k of them (or all that are not minus infinity), best first in the order `distribution` sorts by (larger
    logit, then larger id; an id of -1 ends the list).  The same arithmetic on the same numbers."""
    ids = np.asarray(ids)
    values = np.asarray(values, dtype=np.float32)
    present = int((ids >= 0).sum())
    if present == 0:
        raise ValueError("empty sampling distribution")
    if not 1 <= top_k <= ids.size:
        raise ValueError("the candidates cover a rule that keeps at most as many tokens as there are candidates")
    keep_k = min(top_k, present)
    ids, values = ids[:keep_k], values[:keep_k].astype(np.float64)
    weights = np.exp((values - values[0]) / temperature)
    total = float(weights.sum())
    mass = np.cumsum(weights)
    reach = np.nonzero(mass >= top_p * total)[0]
    keep = int(reach[0]) + 1 if reach.size else ids.size
    weights = weights[:keep]
    return ids[:keep], weights / float(weights.sum())


def nucleus_of_candidates(ids, values, largest: float, total: float, temperature: float, top_p: float):
    """`distribution_arrays` of a rule WITHOUT top_k for a row of which the best candidates are known (as in
    `distribution_of_candidates`) together with the row's largest logit and its whole mass
    total = sum_x exp((x - largest) / temperature), which the device summed in 64-bit (the reference extracts
    candidates and normalisers in the same way: src/gpu/kernels/llama_nucleus.rs:17-124).  Returns None when the
    candidates do not settle it and the whole row is needed: top_p = 1; a kept prefix that is longer than the
    candidates; or a cut so close to top_p * total (within 1e-10 of the total, the margin of
    src/sampling/nucleus.rs:82-88) that another order of summation could place it elsewhere.  Otherwise the same
    tokens and, number for number, the same probabilities as from the whole row."""
    ids = np.asarray(ids)
    values = np.asarray(values, dtype=np.float32)
    present = int((ids >= 0).sum())
    if present == 0:
        raise ValueError("empty sampling distribution")
    if not (math.isfinite(total) and total > 0.0 and math.isfinite(largest)) or float(values[0]) != largest:
        raise ValueError("invalid softmax mass of a row")
    if top_p >= 1.0:
        return None
    weights = np.exp((values[:present].astype(np.float64) - largest) / temperature)
    mass = np.cumsum(weights)
    target = top_p * total
    reach = np.nonzero(mass >= target)[0]
    if not reach.size:
        return None
    keep = int(reach[0]) + 1
    margin = abs(total) * 1e-10
    before = float(mass[keep - 2]) if keep > 1 else 0.0
    if before >= target - margin or float(mass[keep - 1]) <= target + margin:
        return None
    weights = weights[:keep]
    return ids[:keep], weights / float(weights.sum())


class RequestSampler:
    """The sampling state of one request."""

    def __init__(self, params: Sampling):
        self.params = params
        self.random = MT19937(params.seed & 0xFFFFFFFF)
        self.generated = set()

    def penalised(self, logits: np.ndarray) -> np.ndarray:
        if self.params.presence_penalty == 0.0 or not self.generated:
            return logits
        out = np.array(logits, dtype=np.float32, copy=True)
        out[sorted(self.generated)] -= np.float32(self.params.presence_penalty)
        return out

    def sample_candidates(self, ids, values, position: int, mass=None):
        """`sample` for a row of which the device extracted the best candidates (see
        `distribution_of_candidates`): for rules without a presence penalty that are greedy, keep at most len(ids)
        tokens, or (with `mass`, the row's largest logit and whole softmax mass) have no top_k but a top_p below 1.
        The same token as `sample` on the whole row, or None if the candidates do not settle it (no random number
        is drawn then): the caller samples from the whole row."""
        p = self.params
        if p.presence_penalty != 0.0:
            raise ValueError("a presence penalty needs the whole row")
        if p.greedy:
            token = int(ids[0])
        elif p.top_k >= 1:
            token = self._draw(distribution_of_candidates(ids, values, p.temperature, p.top_k, p.top_p), position)
        else:
            if mass is None:
                raise ValueError("a rule without top_k needs the row's softmax mass beside the candidates")
            entries = nucleus_of_candidates(ids, values, float(mass[0]), float(mass[1]), p.temperature, p.top_p)
            if entries is None:
                return None
            token = self._draw(entries, position)
        self.accept(token)
        return token

    def sample(self, logits: np.ndarray, position: int) -> int:
        """Choose from one row of 32-bit logits on the host.  `position` is that of the token
        whose logits these are (it keys the Gumbel noise: src/server/paged/request.rs:114)."""
        p = self.params
        logits = np.asarray(logits, dtype=np.float32)
        if not np.isfinite(logits).all():
            raise ValueError("nonfinite output logits")
        logits = self.penalised(logits)
        if p.greedy:
            best = logits.max()
            token = int(np.nonzero(logits == best)[0].max())
        else:
            token = self._draw(distribution_arrays(logits, p.temperature, p.top_k, p.top_p), position)
        self.accept(token)
        return token

    def _draw(self, entries, position: int) -> int:
        """One token from (tokens, probabilities), best first."""
        p = self.params
        tokens, probabilities = entries
        if p.sampler == "murmur3_gumbel":
            scored = [(np.float32(math.log(prob)) + np.float32(gumbel_noise(murmur_hash(p.seed, position, int(tok)))),
                       -int(tok), int(tok)) for tok, prob in zip(tokens, probabilities)]
            return max(scored)[2]
        if len(tokens) == 1:
            return int(tokens[0])
        # the first entry whose running sum (added up one by one, in order) exceeds the sample; else the last
        beyond = np.searchsorted(np.cumsum(probabilities), self.random.uniform(), side="right")
        return int(tokens[min(int(beyond), len(tokens) - 1)])

    def accept(self, token: int) -> None:
        self.generated.add(int(token))
