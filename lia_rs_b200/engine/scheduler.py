"""The scheduler above the step function: it admits requests, cuts prompts into portions under a
token budget, decodes, finishes and frees, and decides what happens when pages run out.

The policy is the reference's continuous-batching loop (src/server/paged.rs:64-99,
src/server/paged/{request,schedule,preempt}.rs):

* Admission is first come, first served, paused requests before queued ones; a request is
  admitted when a slot is free, its prompt is shorter than the context, and the pages for its
  first token exist; otherwise it stays at the head and admission stops (request.rs:6-24,85-88;
  preempt.rs:5-21).
* Decoding is not a mode of its own: a request with one uncomputed token contributes one row
  (schedule.rs:28-50).  Budget: `max_batch_tokens` rows a step.  By default single decoded tokens
  come first and the rest of the budget goes to prompt portions in slot order; `even_split=True`
  gives every live request max(1, budget / live) rows, as the reference does (schedule.rs:11).
* A portion is shortened where its next page cannot be had (schedule.rs:30-36).
* Before each step, if more requests need a new page than there are free pages, requests are
  preempted until the rest fits: the victim is the one that has already produced its first token,
  then holds most pages, then sits in the highest slot; its pages are given back, it keeps its
  tokens and sampler and is recomputed from position 0 when it is resumed.  A single request that
  cannot fit raises "one request exceeded its physical KV capacity" (preempt.rs:61-113).
* A step in which live requests exist but no row could be scheduled raises
  "active KV scheduler made no progress" (schedule.rs:123-125).
* A request is done at an end-of-sequence token or after `max_tokens` tokens; the last token is not
  fed back (request.rs:128-147).  Its pages and slot are freed at once (schedule.rs:126-137).

Steady decoding is pipelined (`pipeline=True`, with an engine that offers `select_tokens_start`): while every
live request just decodes, nothing waits to be admitted, nobody reaches `max_tokens` and the pages suffice,
`step()` launches the next decode step with the tokens fed on the device and only then reads the tokens of
the step before from the host copy, so the host's bookkeeping runs under the GPU's work.  What the requests
receive does not change.  A request that the token just read ends (end of sequence) has one more token
computed that nobody looks at; its pages are freed when that is known.  Every other situation (a prompt
portion, an admission, a request at its last token, pages running out) first reads what is pending and then
takes the plain path above.
"""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Optional

from ..sampling import RequestSampler, Sampling
from .step import StepEntry


class SchedulerError(RuntimeError):
    pass


@dataclass
class Request:
    rid: object
    prompt: list
    sampling: Sampling
    max_tokens: int
    tokens: list = field(default_factory=list)          # prompt + accepted tokens that are fed back
    generated: list = field(default_factory=list)
    computed: int = 0                                   # tokens whose keys and values are in the cache
    slot: Optional[int] = None
    sampler: Optional[RequestSampler] = None
    done: bool = False
    stopped: bool = False                               # ended by an end-of-sequence token
    error: Optional[str] = None
    preemptions: int = 0
    submitted: float = 0.0
    first_token: Optional[float] = None
    finished: Optional[float] = None


class Scheduler:
    NUCLEUS_CANDIDATES = 32                              # candidates asked of the device for a rule without top_k

    def __init__(self, engine, max_batch_tokens: int = 512, even_split: bool = False, eos_token_ids=(),
                 context: Optional[int] = None, pipeline: bool = True):
        self.engine = engine
        self.cache = engine.cache
        self.budget = int(max_batch_tokens)
        if self.budget <= 0:
            raise SchedulerError("max_batch_tokens must be positive")
        self.even_split = even_split
        self.eos = set(int(t) for t in eos_token_ids)
        self.context = int(context or self.cache.max_context)
        self.queue, self.paused = deque(), deque()
        self.active = [None] * self.cache.max_slots      # by slot
        self.finished = []
        self.stats = {"steps": 0, "preemptions": 0, "prefill_tokens": 0, "decode_tokens": 0, "admitted": 0,
                      "pipelined_steps": 0, "candidate_steps": 0, "whole_row_draws": 0}
        self.pipeline = bool(pipeline) and hasattr(engine, "select_tokens_start")
        self._pending = None                             # (tokens on their way to the host, the requests they belong to)

    # ---- requests ----
    def add(self, rid, prompt, sampling: Sampling = None, max_tokens: int = 8192) -> Request:
        """Queue a request.  `max_tokens` is clamped to context - prompt (request.rs:40-48)."""
        prompt = [int(t) for t in prompt]
        request = Request(rid, prompt, sampling or Sampling(), int(max_tokens), tokens=list(prompt),
                          submitted=time.perf_counter())
        request.sampler = RequestSampler(request.sampling)
        if not prompt or len(prompt) >= self.context:
            request.error, request.done = "prompt exceeds request context", True
            self.finished.append(request)
            return request
        request.max_tokens = min(request.max_tokens, self.context - len(prompt))
        if request.max_tokens <= 0:
            request.error, request.done = "completion token limit must be positive", True
            self.finished.append(request)
            return request
        self.queue.append(request)
        return request

    def has_work(self) -> bool:
        return bool(self.queue or self.paused or any(r is not None for r in self.active))

    def live(self) -> list:
        return [r for r in self.active if r is not None]

    # ---- admission ----
    def _attach(self, request: Request) -> bool:
        """A slot and the page of the first uncomputed token, or nothing."""
        if self.cache.free_slots() == 0:
            return False
        slot = self.cache.admit()
        if not self.cache.ensure(slot, 0, 1):
            self.cache.release(slot)
            return False
        request.slot, request.computed = slot, 0
        self.active[slot] = request
        return True

    def admit(self) -> None:
        while self.cache.free_slots() > 0:
            if self.paused:
                request = self.paused[0]
                # do not take a paused request back before its whole prefix fits again (preempt.rs:38-42)
                needed = (len(request.tokens) + self.cache.page_size - 1) // self.cache.page_size
                if needed > self.cache.available_pages() or not self._attach(request):
                    return
                self.paused.popleft()
                continue
            if not self.queue:
                return
            if not self._attach(self.queue[0]):
                return
            self.queue.popleft()
            self.stats["admitted"] += 1

    # ---- pages run out ----
    def _needs_new_page(self, request: Request) -> bool:
        return (not request.done) and self.cache.pages_for(request.slot, request.computed, request.computed + 1) > 0

    def pause_for_capacity(self) -> None:
        while True:
            live = self.live()
            needed = sum(1 for r in live if self._needs_new_page(r))
            if needed <= self.cache.available_pages():
                return
            if len(live) <= 1:
                raise SchedulerError("one request exceeded its physical KV capacity")
            victim = max(live, key=lambda r: (bool(r.generated), self._pages_held(r), r.slot))
            self._preempt(victim)

    def _pages_held(self, request: Request) -> int:
        return max(group.held_by(request.slot) for group in self.cache.groups) \
            if self.cache.groups else 0

    def _preempt(self, request: Request) -> None:
        self.cache.release(request.slot)
        self.active[request.slot] = None
        request.slot, request.computed = None, 0
        request.preemptions += 1
        self.paused.append(request)
        self.stats["preemptions"] += 1

    # ---- one step ----
    def _portion(self, request: Request, allowance: int) -> int:
        """How many of the request's next tokens (at most `allowance`) have pages; the portion is
        cut at the first page that cannot be had."""
        start = request.computed
        want = min(allowance, len(request.tokens) - start)
        while want > 0 and not self.cache.ensure(request.slot, start, start + want):
            # shorten to the end of the last page that can still be had
            ps = self.cache.page_size
            boundary = ((start + want - 1) // ps) * ps
            want = boundary - start if boundary > start else 0
        return want

    def plan(self) -> list:
        """[(request, count)] for this step, pages reserved."""
        live = self.live()
        if not live:
            return []
        plan, budget = [], self.budget
        if self.even_split:
            allowance = max(1, self.budget // len(live))
            for request in live:
                count = self._portion(request, allowance)
                if count:
                    plan.append((request, count))
            return plan
        decoding = [r for r in live if len(r.tokens) - r.computed == 1]
        prefilling = [r for r in live if len(r.tokens) - r.computed > 1]
        for request in decoding:
            if budget <= 0:
                break
            if self._portion(request, 1):
                plan.append((request, 1))
                budget -= 1
        for request in prefilling:
            if budget <= 0:
                break
            count = self._portion(request, budget)
            if count:
                plan.append((request, count))
                budget -= count
        return plan

    def step(self) -> list:
        """Admit, make room, run one batch, sample, finish.  Returns the requests that finished (with
        `pipeline`, those whose last token this call read: it may belong to the step before)."""
        done = []
        if self._pending is not None:
            if self._can_continue():
                following = self._launch_fed()           # the GPU goes on ...
                done = self._collect()                   # ... while the host reads the step before
                self._pending = following
                return done
            done = self._collect()
        self.admit()
        self.pause_for_capacity()
        plan = self.plan()
        live = self.live()
        if not plan:
            if any(not r.done for r in live):
                raise SchedulerError("active KV scheduler made no progress")
            return done
        entries, outputs = [], []
        for request, count in plan:
            start = request.computed
            last = start + count == len(request.tokens)
            entries.append(StepEntry(request.slot, request.tokens[start:start + count], start,
                                     [count - 1] if last else []))
            if last:
                outputs.append(request)
            if count > 1 or start + count < len(request.prompt):
                self.stats["prefill_tokens"] += count
            else:
                self.stats["decode_tokens"] += count
        logits = self.engine.step(entries)
        for request, count in plan:
            request.computed += count
        self.stats["steps"] += 1
        if outputs:
            if self.pipeline and all(r.sampling.on_device for r in outputs):
                self._pending = (self._select_start(logits, outputs), outputs)
                return done
            tokens = self._select(logits, outputs)
            now = time.perf_counter()
            for request, token in zip(outputs, tokens):
                self._accept(request, int(token), now)
        return done + self._retire()

    def _retire(self) -> list:
        """Free what the finished requests hold."""
        done = []
        for request in self.live():
            if request.done:
                self.cache.release(request.slot)
                self.active[request.slot] = None
                request.slot = None
                request.finished = time.perf_counter()
                done.append(request)
        self.finished.extend(done)
        return done

    # ---- pipelined decoding ----
    def _select_start(self, logits, requests):
        return self.engine.select_tokens_start(logits, [r.sampling for r in requests], [r.computed - 1 for r in requests])

    def _collect(self) -> list:
        """Read the pending tokens, give them to their requests, retire the finished."""
        pending, requests = self._pending
        self._pending = None
        tokens = pending.tokens()
        now = time.perf_counter()
        for request, token in zip(requests, tokens):
            if request.done:                             # ended a step ago: this token was computed for nobody
                continue
            request.sampler.accept(int(token))
            self._accept(request, int(token), now)
        return self._retire()

    def _can_continue(self) -> bool:
        """Whether the step after the pending one is known before its tokens are: every live request decodes
        on, whatever token it gets (short of an end of sequence)."""
        _, requests = self._pending
        live = self.live()
        if self.queue or self.paused or len(live) != len(requests) or len(live) > self.budget:
            return False
        needed = 0
        for request, other in zip(live, requests):
            if request is not other or request.done or len(request.tokens) != request.computed:
                return False
            if len(request.generated) + 1 >= request.max_tokens:        # the pending token is its last
                return False
            needed += self.cache.pages_for(request.slot, request.computed, request.computed + 1) > 0
        return needed <= self.cache.available_pages()

    def _launch_fed(self):
        """The next decode step of the pending step's requests, their tokens taken on the device."""
        pending, requests = self._pending
        entries = []
        for request in requests:
            if not self.cache.ensure(request.slot, request.computed, request.computed + 1):
                raise SchedulerError("a page that was counted free could not be had")
            entries.append(StepEntry(request.slot, [0], request.computed, [0]))
        logits = self.engine.step(entries, feed=pending)
        for request in requests:
            request.computed += 1
        self.stats["steps"] += 1
        self.stats["pipelined_steps"] += 1
        self.stats["decode_tokens"] += len(requests)
        return (self._select_start(logits, requests), requests)

    def _select(self, logits, requests) -> list:
        """One token per output row: on the device where the rule allows it, else on the host."""
        positions = [r.computed - 1 for r in requests]
        if all(r.sampling.on_device for r in requests):
            tokens = self.engine.select_tokens(logits, [r.sampling for r in requests], positions)
            for request, token in zip(requests, tokens):
                request.sampler.accept(int(token))
            return tokens
        # rules that keep at most top_k tokens (and greedy ones) need only the row's best candidates, which the
        # device extracts: a few hundred bytes to the host instead of the rows.  A rule without top_k but with
        # top_p < 1 takes the best candidates too, and the row's whole softmax mass: when its kept tokens lie
        # within them it draws from them, else from the whole row (the reference's extraction of candidates and
        # normalisers with its fall-back, src/gpu/kernels/llama_nucleus.rs:17-124, src/sampling/nucleus.rs:48-91)
        rules = [r.sampling for r in requests]
        open_ended = [not s.greedy and s.top_k == 0 for s in rules]
        if hasattr(self.engine, "select_candidates") and all(
                s.presence_penalty == 0.0 and (s.greedy or s.top_k >= 1 or s.top_p < 1.0) for s in rules):
            k = max([s.top_k for s in rules if not s.greedy] + [self.NUCLEUS_CANDIDATES if any(open_ended) else 1])
            self.stats["candidate_steps"] += 1
            if any(open_ended):
                values, ids, mass = self.engine.select_candidates(
                    logits, k, [s.temperature if o else 0.0 for s, o in zip(rules, open_ended)])
            else:
                (values, ids), mass = self.engine.select_candidates(logits, k), [None] * len(requests)
            tokens = [r.sampler.sample_candidates(ids[i], values[i], positions[i], mass[i]) for i, r in enumerate(requests)]
            if any(t is None for t in tokens):
                rows = self.engine.logits_to_host(logits)
                for i, r in enumerate(requests):
                    if tokens[i] is None:
                        self.stats["whole_row_draws"] += 1
                        tokens[i] = r.sampler.sample(rows[i], positions[i])
            return tokens
        rows = self.engine.logits_to_host(logits)
        return [r.sampler.sample(rows[i], positions[i]) for i, r in enumerate(requests)]

    def _accept(self, request: Request, token: int, now: float) -> None:
        if request.first_token is None:
            request.first_token = now
        request.generated.append(token)
        request.stopped = token in self.eos
        request.done = request.stopped or len(request.generated) >= request.max_tokens
        if not request.done:
            request.tokens.append(token)

    def run(self) -> list:
        """Step until nothing is left; returns all finished requests in the order they finished."""
        while self.has_work():
            self.step()
        return self.finished
