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
"""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Optional

import numpy as np

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
    def __init__(self, engine, max_batch_tokens: int = 512, even_split: bool = False, eos_token_ids=(),
                 context: Optional[int] = None):
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
        self.stats = {"steps": 0, "preemptions": 0, "prefill_tokens": 0, "decode_tokens": 0, "admitted": 0}

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
        return max(sum(1 for p in group.tables[request.slot] if p >= 0) for group in self.cache.groups) \
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
        """Admit, make room, run one batch, sample, finish.  Returns the requests that finished in
        this step."""
        self.admit()
        self.pause_for_capacity()
        plan = self.plan()
        live = self.live()
        if not plan:
            if any(not r.done for r in live):
                raise SchedulerError("active KV scheduler made no progress")
            return []
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
        if outputs:
            tokens = self._select(logits, outputs)
            now = time.perf_counter()
            for request, token in zip(outputs, tokens):
                self._accept(request, int(token), now)
        self.stats["steps"] += 1
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

    def _select(self, logits, requests) -> list:
        """One token per output row: on the device where the rule allows it, else on the host."""
        positions = [r.computed - 1 for r in requests]
        if all(r.sampling.on_device for r in requests):
            tokens = self.engine.select_tokens(logits, [r.sampling for r in requests], positions)
            for request, token in zip(requests, tokens):
                request.sampler.accept(int(token))
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
