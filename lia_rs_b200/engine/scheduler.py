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

import ctypes
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Optional

from ..cache.pages import host_library
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
    number: int = -1                                     # the native core's name for the request


class Scheduler:
    """The face of the native policy (csrc/host/scheduler_host.cpp): it owns the requests' tokens, samplers and
    times, asks the native core whom to admit, whom to preempt and what a step runs, runs the step and reports
    what was accepted.  `queue`, `paused`, `active` and a request's `slot`, `computed` and `preemptions` mirror
    the core's state."""
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
        self._lib = host_library()
        self._lib.lia_sched_create.restype = ctypes.c_void_p
        self._core = ctypes.c_void_p(self._lib.lia_sched_create(self.cache._handle, self.budget, int(bool(even_split)),
                                                                self.cache.max_context, self.cache.page_size))
        if not self._core:
            raise SchedulerError(self._lib.lia_host_error().decode())
        self._requests = []                              # by the core's request number
        self._events = (ctypes.c_int * (3 * (2 * self.cache.max_slots + 2)))()
        self._plan = (ctypes.c_int * (4 * self.cache.max_slots))()
        self._retired = (ctypes.c_int * self.cache.max_slots)()

    def __del__(self):
        core, self._core = getattr(self, "_core", None), None
        if core:
            self._lib.lia_sched_destroy(core)

    def _refused(self):
        raise SchedulerError(self._lib.lia_host_error().decode())

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
        request.number = self._lib.lia_sched_add(self._core, len(prompt), request.max_tokens)
        if request.number < 0:
            self._refused()
        self._requests.append(request)
        self.queue.append(request)
        return request

    def core_state(self, request: Request) -> dict:
        """What the native core holds of a request (a test compares it with the face's mirror)."""
        out = (ctypes.c_int * 6)()
        if self._lib.lia_sched_request(self._core, request.number, out) < 0:
            self._refused()
        return dict(slot=None if out[0] < 0 else out[0], computed=out[1], tokens=out[2], generated=out[3],
                    done=bool(out[4]), preemptions=out[5])

    def has_work(self) -> bool:
        return bool(self.queue or self.paused or any(r is not None for r in self.active))

    def live(self) -> list:
        return [r for r in self.active if r is not None]

    # ---- admission, and what happens when pages run out ----
    def prepare(self) -> None:
        """Admission (first come, first served, paused requests first), then room for the step: while more live
        requests need a new page than pages are free, one is preempted.  The core decides; what it did is taken
        over here."""
        n = self._lib.lia_sched_prepare(self._core, self._events, len(self._events) // 3)
        if n < 0:
            self._refused()
        for i in range(n):
            kind, number, slot = self._events[3 * i:3 * i + 3]
            request = self._requests[number]
            if kind == 2:                                # preempted: its pages are back, it waits to be computed again
                self.active[slot] = None
                request.slot, request.computed = None, 0
                request.preemptions += 1
                self.paused.append(request)
                self.stats["preemptions"] += 1
                continue
            waiting = self.queue if kind == 1 else self.paused
            assert waiting[0] is request
            waiting.popleft()
            request.slot, request.computed = slot, 0
            self.active[slot] = request
            self.cache.admitted(slot)
            if kind == 1:
                self.stats["admitted"] += 1

    # ---- one step ----
    def plan(self) -> list:
        """[(request, count)] for this step, pages reserved: single decoded tokens first, then prompt portions in
        slot order under the budget (or the even split), each portion cut at the first page that cannot be had."""
        n = self._lib.lia_sched_plan(self._core, self._plan, len(self._plan) // 4)
        if n < 0:
            self._refused()
        return [(self._requests[self._plan[4 * i]], self._plan[4 * i + 2]) for i in range(n)]

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
        self.prepare()
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
            self._advance(request, count)
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

    def _advance(self, request: Request, count: int) -> None:
        if self._lib.lia_sched_advance(self._core, request.number, count) < 0:
            self._refused()
        request.computed += count

    def _retire(self) -> list:
        """Free what the finished requests hold."""
        n = self._lib.lia_sched_retire(self._core, self._retired)
        if n < 0:
            self._refused()
        done = []
        for number in self._retired[:n]:
            request = self._requests[number]
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
        numbers = (ctypes.c_int * max(1, len(requests)))(*[r.number for r in requests])
        answer = self._lib.lia_sched_can_continue(self._core, numbers, len(requests))
        if answer < 0:
            self._refused()
        return bool(answer)

    def _launch_fed(self):
        """The next decode step of the pending step's requests, their tokens taken on the device."""
        pending, requests = self._pending
        numbers = (ctypes.c_int * max(1, len(requests)))(*[r.number for r in requests])
        if self._lib.lia_sched_reserve_next(self._core, numbers, len(requests)) < 0:
            self._refused()
        entries = [StepEntry(request.slot, [0], request.computed, [0]) for request in requests]
        logits = self.engine.step(entries, feed=pending)
        for request in requests:
            self._advance(request, 1)
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
        if self._lib.lia_sched_accept(self._core, request.number, int(request.done)) < 0:
            self._refused()
        if not request.done:
            request.tokens.append(token)

    def run(self) -> list:
        """Step until nothing is left; returns all finished requests in the order they finished."""
        while self.has_work():
            self.step()
        return self.finished
