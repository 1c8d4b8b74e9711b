"""The scheduler: admits requests, cuts prompts into portions under a token
budget, lets every running request decode, finishes and frees.

The reference admits every queued request whose prompt (plus one token) fits
the free pages, prefills it whole and alone, then decodes all active sequences
in one forward (engine/llama_paged_engine.py:418-442).  It has no token budget,
and when a decode step needs a page that is not there the engine loop dies
with an exception (:276, engine/paged_cache.py:51-55); a prompt larger than the
pool spins forever (:453).

Decisions here:
  * a step carries at most ``max_tokens_per_step`` tokens: first one token for
    every request that is decoding, then portions of prompts, oldest first, at
    most ``chunk`` tokens of one request;
  * requests are admitted first come, first served, while a request slot and
    the pages of the whole prompt plus one token are free beyond what running
    prompts still need;
  * a request that can never fit (prompt + max_new_tokens beyond the pool or the
    model's positions) is refused at ``submit``;
  * when a decoding request needs a page and none is free, the YOUNGEST running
    request is preempted: its pages and slot go back, and it returns to the
    head of the queue to be recomputed from its prompt and what it generated;
    the loop never raises for lack of pages.

This file is host logic only and runs without a GPU.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable

from ..sampling.sampler import SamplingConfig


@dataclass
class Request:
    """A generation request; the fields of engine/llama_paged_engine.py:85-103
    plus per-request sampling."""

    req_id: int
    prompt_ids: list[int]
    max_new_tokens: int
    arrival_time: float = 0.0
    generated: list[int] = field(default_factory=list)
    start_time: float = 0.0
    finish_time: float = 0.0
    stop_check: Callable[[list[int]], bool] | None = field(default=None, repr=False)
    sampling: SamplingConfig | None = None
    error: str | None = None
    preemptions: int = 0

    @property
    def job_size(self) -> int:
        return len(self.prompt_ids) + self.max_new_tokens

    @property
    def tokens(self) -> list[int]:
        return self.prompt_ids + self.generated

    # the reference keeps the three time stamps (engine/llama_paged_engine.py:92-95) and leaves the figures to its caller
    @property
    def ttft(self) -> float | None:
        """Seconds from arrival to the first generated token (None until there is one)."""
        return self.start_time - self.arrival_time if self.start_time else None

    @property
    def tpot(self) -> float | None:
        """Seconds per generated token after the first (None unless finished with at least two)."""
        if not self.finish_time or len(self.generated) < 2:
            return None
        return (self.finish_time - self.start_time) / (len(self.generated) - 1)


PLACEHOLDER = -1    # stands in ``generated`` for a token that was sampled on the device and not read yet


@dataclass
class PlannedEntry:
    request: Request
    tokens: list[int]
    wants_logits: bool
    slot: int = -1           # index in ``generated`` of the token this entry samples (booked steps)
    last: bool = False       # the request ends with this token whatever it is (max_new_tokens)
    cancelled: bool = False  # the request ended at an earlier token: this entry's result is dropped


@dataclass
class StepPlan:
    entries: list[PlannedEntry]
    preempted: list[Request]
    admitted: list[Request]

    @property
    def n_tokens(self) -> int:
        return sum(len(e.tokens) for e in self.entries)


class Scheduler:
    def __init__(self, cache, max_positions: int, max_batch: int = 64, max_tokens_per_step: int = 2048,
                 chunk: int | None = None, max_queue_depth: int = 4096, eos_token=None):
        if max_tokens_per_step < 1:
            raise ValueError("max_tokens_per_step must be at least 1")
        self.cache = cache
        self.max_positions = max_positions
        self.max_batch = min(max_batch, cache.max_requests)
        self.max_tokens_per_step = max_tokens_per_step
        self.chunk = chunk or max_tokens_per_step
        self.max_queue_depth = max_queue_depth
        self.eos = set(eos_token) if isinstance(eos_token, (tuple, list, set)) else ({eos_token} if eos_token is not None else set())
        self.queue: list[Request] = []
        self.running: list[Request] = []          # in order of admission, oldest first
        self.completed: list[Request] = []
        self.n_preemptions = 0

    # ------------------------------------------------------------------ intake
    def submit(self, req: Request) -> bool:
        """Enqueue; False (and ``req.error`` set) if the queue is full or the request can never fit."""
        if len(self.queue) >= self.max_queue_depth:
            req.error = "queue full"
            return False
        if not req.prompt_ids:
            req.error = "empty prompt"
            return False
        total = len(req.prompt_ids) + max(req.max_new_tokens, 0)
        if total > self.max_positions:
            req.error = f"prompt + max_new_tokens = {total} exceeds the model's {self.max_positions} positions"
            return False
        ps = self.cache.page_size
        if -(-total // ps) > min(self.cache.n_pages, self.cache.max_pages_per_request):
            req.error = f"prompt + max_new_tokens = {total} tokens can never fit the cache pool"
            return False
        self.queue.append(req)
        return True

    @property
    def has_work(self) -> bool:
        return bool(self.queue) or bool(self.running)

    # ---------------------------------------------------------------- planning
    def _remaining(self, req: Request) -> int:
        return len(req.prompt_ids) + len(req.generated) - self.cache.lengths[req.req_id]

    def _pages_for(self, n_tokens: int) -> int:
        return -(-n_tokens // self.cache.page_size)

    def _preempt(self, req: Request, plan: StepPlan) -> None:
        self.cache.close(req.req_id)
        self.running.remove(req)
        req.preemptions += 1
        self.n_preemptions += 1
        self.queue.insert(0, req)
        plan.preempted.append(req)
        plan.entries = [e for e in plan.entries if e.request is not req]

    def plan(self) -> StepPlan:
        """Decide the next step and reserve its pages."""
        plan = StepPlan([], [], [])
        while True:
            self._plan_once(plan)
            if plan.entries or not self.running:
                return plan
            # every running request is stuck behind pages that others hold: the youngest gives way
            self._preempt(self.running[-1], plan)

    def _plan_once(self, plan: StepPlan) -> None:
        cache = self.cache
        budget = self.max_tokens_per_step
        planned = set()

        # 1. one token for every request that is decoding, oldest first
        i = 0
        while i < len(self.running) and budget > 0:
            req = self.running[i]
            if self._remaining(req) != 1:
                i += 1
                continue
            new_len = cache.lengths[req.req_id] + 1
            ok = cache.reserve(req.req_id, new_len)
            while not ok:
                victim = self.running[-1]
                self._preempt(victim, plan)
                planned.discard(victim.req_id)
                if victim is req:
                    break
                ok = cache.reserve(req.req_id, new_len)
            if ok:
                plan.entries.append(PlannedEntry(req, [req.tokens[-1]], True))
                planned.add(req.req_id)
                budget -= 1
                i += 1
            # else ``req`` itself gave way and running[i] is already the next request

        # 2. portions of prompts of running requests, oldest first
        for req in list(self.running):
            if budget <= 0:
                break
            if req.req_id in planned:
                continue
            rem = self._remaining(req)
            if rem >= 1:
                took = self._plan_portion(req, rem, budget, plan)
                budget -= took
                if took:
                    planned.add(req.req_id)

        # 3. admissions, first come first served
        while self.queue and budget > 0 and len(self.running) < self.max_batch and cache.n_free_slots > 0:
            req = self.queue[0]
            n_all = len(req.prompt_ids) + len(req.generated)
            promised = sum(max(0, self._pages_for(len(r.prompt_ids) + len(r.generated) + 1)
                               - self._pages_for(cache.reserved[r.req_id])) for r in self.running)
            if cache.n_free_pages() - promised < self._pages_for(n_all + 1):
                break
            self.queue.pop(0)
            slot = cache.open(req.req_id)
            assert slot is not None
            self.running.append(req)
            plan.admitted.append(req)
            took = self._plan_portion(req, n_all, budget, plan)
            budget -= took
            if took == 0:
                break

    def _plan_portion(self, req: Request, remaining: int, budget: int, plan: StepPlan) -> int:
        """Plan up to min(remaining, chunk, budget) further tokens of ``req``; shrink to the pages that are free."""
        cache = self.cache
        base = cache.lengths[req.req_id]
        n = min(remaining, self.chunk, budget)
        while n > 0 and not cache.reserve(req.req_id, base + n):
            # shrink to a page boundary that might fit
            fit = (cache.n_free_pages() + self._pages_for(cache.reserved[req.req_id])) * cache.page_size - base
            n = min(n - 1, max(0, fit))
        if n <= 0:
            return 0
        toks = req.tokens[base:base + n]
        plan.entries.append(PlannedEntry(req, toks, wants_logits=(n == remaining)))
        return n

    # --------------------------------------------------------------- after a step
    def commit(self, plan: StepPlan, sampled: dict, now: float = 0.0) -> list[Request]:
        """Record the step's sampled tokens (``{req_id: token}`` for the entries that
        wanted logits); finish and free what is done.  Returns the requests finished."""
        finished = []
        for e in plan.entries:
            req = e.request
            if not e.wants_logits:
                continue
            tok = int(sampled[req.req_id])
            if not req.generated or req.start_time == 0.0:
                req.start_time = req.start_time or now
            req.generated.append(tok)
            # engine/llama_paged_engine.py:207-211, 267-271: the EOS token is kept in ``generated``
            done = (len(req.generated) >= req.max_new_tokens or tok in self.eos
                    or (req.stop_check is not None and req.stop_check(req.generated)))
            if done:
                req.finish_time = now
                self.cache.close(req.req_id)
                self.running.remove(req)
                self.completed.append(req)
                finished.append(req)
        return finished

    # ------------------------------------------------- steps booked before their tokens are read
    def book(self, plan: StepPlan) -> None:
        """Record a step that has been enqueued while its sampled tokens are still on the device: every
        sampling entry gets a PLACEHOLDER in ``generated``; a request that reaches ``max_new_tokens`` ends
        here and gives its pages back (later steps run after this one on the device, so the pages are not
        rewritten before it has finished)."""
        for e in plan.entries:
            if not e.wants_logits:
                continue
            req = e.request
            e.slot = len(req.generated)
            req.generated.append(PLACEHOLDER)
            if len(req.generated) >= req.max_new_tokens:
                e.last = True
                self.cache.close(req.req_id)
                self.running.remove(req)

    def resolve(self, plan: StepPlan, sampled: dict, in_flight: StepPlan | None = None, now: float = 0.0) -> list[Request]:
        """The tokens of a booked step have arrived: put them in place of the placeholders, and end the
        requests that end with them (EOS, stop_check, or booked as last).  A request that ends by its token
        may have an entry in the step ``in_flight``; that entry is cancelled and its placeholder dropped."""
        finished = []
        for e in plan.entries:
            if not e.wants_logits or e.cancelled:
                continue
            req = e.request
            tok = int(sampled[req.req_id])
            req.generated[e.slot] = tok
            req.start_time = req.start_time or now
            by_token = tok in self.eos or (req.stop_check is not None and req.stop_check(req.generated[:e.slot + 1]))
            if not (e.last or by_token):
                continue
            if by_token:
                del req.generated[e.slot + 1:]
                if in_flight is not None:
                    for f in in_flight.entries:
                        if f.request is req:
                            f.cancelled = True
                if req in self.running:
                    self.cache.close(req.req_id)
                    self.running.remove(req)
            req.finish_time = now
            self.completed.append(req)
            finished.append(req)
        return finished
