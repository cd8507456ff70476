"""Continuous batching: which requests run in the next step, and with how many tokens.

Host-only decisions, after upstream's ``Scheduler`` (server.py:101-292): a FIFO queue,
a list of active requests, admission by one of two page plans, newest-first preemption
with recomputation when pages run out.  What is different: a step has a token budget,
prompts are cut into portions under it, and portions of prompts run in the same step as
the single tokens of decoding requests (upstream prefills whole prompts in launches of
their own, server.py:279-284, 329).

Pages run out — what happens (decided here, tested in tests/test_scheduler.py):

1. Decoding requests come first.  While the pages their next tokens need exceed the free
   pages, the newest active request is preempted: its pages and slot are given back, it
   returns to the *front* of the queue, and when admitted again it is fed its prompt and
   everything it generated so far (upstream ``preempt``, server.py:187-193).
2. Prompt portions are elastic: a portion is cut down to the tokens that fit the pages
   still free (and the token budget); a request that gets nothing waits for a later step.
3. If a step would run nothing and more than one request is active, the newest is
   preempted and the plan is made again.  If the only active request cannot take a
   single token, the pool is too small for it: ``PoolTooSmall`` (upstream's
   ``RuntimeError("kv pool too small for a single request")``, server.py:267-268).
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, List, Optional, Sequence

from ..sampling.params import SamplingParams


class PoolTooSmall(RuntimeError):
    pass


class Request:
    """One generation request (upstream ``Request``, server.py:76-98)."""
    _next_id = 0

    def __init__(self, prompt_ids: Sequence[int], params: Optional[SamplingParams] = None):
        if len(prompt_ids) == 0:
            raise ValueError("a request needs at least one prompt token")
        self.id = Request._next_id
        Request._next_id += 1
        self.ids: List[int] = [int(t) for t in prompt_ids]   # prompt + generated
        self.prompt_len = len(self.ids)
        self.params = params or SamplingParams()
        self.slot: Optional[int] = None
        self.fed = 0                  # tokens whose keys and values are in the cache
        self.done = False
        self.finish_reason: Optional[str] = None
        self.preempted = 0

    def out_ids(self) -> List[int]:
        return self.ids[self.prompt_len:]

    @property
    def remaining(self) -> int:
        return len(self.ids) - self.fed


@dataclass
class PlannedEntry:
    request: Request
    n_tokens: int
    sample: bool                       # the portion reaches the request's last token


@dataclass
class StepPlan:
    entries: List[PlannedEntry] = field(default_factory=list)
    preempted: List[Request] = field(default_factory=list)

    @property
    def tokens(self) -> int:
        return sum(e.n_tokens for e in self.entries)


class Scheduler:
    def __init__(self, cache, *, max_batch: int, max_tokens_per_step: int, max_context: int,
                 admission: str = "final", eos_token_id: Optional[int] = None):
        if admission not in ("final", "cur"):
            raise ValueError(f"admission must be 'final' or 'cur', got {admission!r}")
        self.cache = cache
        self.max_batch = max_batch
        self.max_tokens_per_step = max_tokens_per_step
        self.max_context = max_context
        self.admission = admission
        self.eos_token_id = eos_token_id
        self.queue: Deque[Request] = deque()
        self.active: List[Request] = []
        self.finished: List[Request] = []
        # counters (upstream: server.py:123-129)
        self.preempts = 0
        self.replays = 0
        self.peak_running = 0
        self.steps = 0
        self.tokens_run = 0
        self.min_free_pages = cache.num_pages

    # ---- queue ------------------------------------------------------------------------
    def submit(self, req: Request) -> None:
        page = self.cache.page_size
        if req.prompt_len >= self.max_context:
            raise ValueError(f"prompt of {req.prompt_len} tokens does not fit the context limit {self.max_context}")
        if self.cache.pages_for_tokens(req.prompt_len + 1) > self.cache.num_pages:
            raise PoolTooSmall(f"prompt of {req.prompt_len} tokens needs "
                               f"{self.cache.pages_for_tokens(req.prompt_len + 1)} pages of {page}; "
                               f"the pool has {self.cache.num_pages}")
        self.queue.append(req)

    def has_work(self) -> bool:
        return bool(self.queue or self.active)

    # ---- admission (upstream admit, server.py:138-168) ------------------------------
    def final_pages(self, r: Request) -> int:
        """Pages the request holds once it has generated all it may."""
        return self.cache.pages_for_tokens(min(r.prompt_len + r.params.max_new_tokens, self.max_context))

    def grow_pages(self, r: Request, n_tokens: int) -> int:
        return self.cache.pages_needed(r.slot, n_tokens)

    def admit(self) -> List[Request]:
        admitted = []
        if not self.queue:
            return admitted
        budget = self.cache.free_pages() - sum(self.grow_pages(r, 1) for r in self.active if r.remaining == 1)
        while self.queue and len(self.active) < self.max_batch and self.cache.has_free_slot():
            q = self.queue[0]
            if self.admission == "final":
                proj = sum(self.final_pages(r) for r in self.active) + self.final_pages(q)
                if proj > self.cache.num_pages and self.active:
                    break
            else:
                need = self.cache.pages_for_tokens(len(q.ids))
                if need > budget and self.active:
                    break
                budget -= need
            self.queue.popleft()
            q.slot = self.cache.admit()
            q.fed = 0
            self.active.append(q)
            admitted.append(q)
        return admitted

    # ---- preemption (upstream preempt, server.py:187-193) ---------------------------
    def _preempt_newest(self, plan: StepPlan) -> None:
        req = self.active.pop()
        self.preempts += 1
        if req.fed > 0:
            self.replays += 1
        self.cache.release(req.slot)
        req.slot = None
        req.fed = 0
        req.preempted += 1
        self.queue.appendleft(req)
        plan.preempted.append(req)

    # ---- the plan of one step -----------------------------------------------------------
    def plan_step(self) -> StepPlan:
        plan = StepPlan()
        while self.active:
            plan.entries = []
            decoding = [r for r in self.active if r.remaining == 1 and r.fed > 0]
            filling = [r for r in self.active if not (r.remaining == 1 and r.fed > 0)]
            need = sum(self.grow_pages(r, 1) for r in decoding)
            if need > self.cache.free_pages():
                if len(self.active) == 1:
                    raise PoolTooSmall("kv pool too small for a single request")
                self._preempt_newest(plan)
                continue
            free = self.cache.free_pages() - need
            budget = self.max_tokens_per_step
            for r in decoding:
                if budget <= 0:
                    break
                plan.entries.append(PlannedEntry(r, 1, True))
                budget -= 1
            for r in filling:
                if budget <= 0:
                    break
                n = min(r.remaining, budget)
                # cut the portion down to the pages that are free
                while n > 0 and self.grow_pages(r, n) > free:
                    fit = (self.cache.pages_held(r.slot) + free) * self.cache.page_size - r.fed
                    n = min(n - 1, max(0, fit))
                if n <= 0:
                    continue
                free -= self.grow_pages(r, n)
                budget -= n
                plan.entries.append(PlannedEntry(r, n, n == r.remaining))
            if plan.entries:
                break
            if len(self.active) == 1:
                raise PoolTooSmall("kv pool too small for a single request")
            self._preempt_newest(plan)
        self.peak_running = max(self.peak_running, len(self.active))
        return plan

    # ---- after the step -------------------------------------------------------------------
    def commit(self, plan: StepPlan, sampled: Sequence[int]) -> List[Request]:
        """Account for a step that ran ``plan``; ``sampled`` holds one token for every entry
        with ``sample`` set, in order.  Returns the requests that finished."""
        it = iter(sampled)
        for e in plan.entries:
            r = e.request
            r.fed += e.n_tokens
            if e.sample:
                r.ids.append(int(next(it)))
                self._finish_check(r)
        self.steps += 1
        self.tokens_run += plan.tokens
        self.min_free_pages = min(self.min_free_pages, self.cache.free_pages())
        done = [r for r in self.active if r.done]
        for r in done:
            self.cache.release(r.slot)
            r.slot = None
            self.finished.append(r)
        self.active = [r for r in self.active if not r.done]
        return done

    def _finish_check(self, r: Request) -> None:
        """Upstream ``finish_check`` (server.py:242-252): end-of-sequence token, the cap on new
        tokens, the context limit."""
        out = r.out_ids()
        eos = self.eos_token_id
        if eos is not None and not r.params.ignore_eos and out and out[-1] == eos:
            r.done, r.finish_reason = True, "eos"
        elif len(out) >= r.params.max_new_tokens:
            r.done, r.finish_reason = True, "length"
        elif len(r.ids) >= self.max_context:
            r.done, r.finish_reason = True, "context"

    def stats(self) -> dict:
        return dict(steps=self.steps, tokens_run=self.tokens_run, preempts=self.preempts, replays=self.replays,
                    peak_running=self.peak_running, min_free_pages=self.min_free_pages,
                    finished=len(self.finished), queued=len(self.queue), active=len(self.active))
