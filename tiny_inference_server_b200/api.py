"""The Python entry point: ``Engine`` — submit requests, step, run, ``generate``.

Upstream's entry is ``Scheduler.submit`` + ``Scheduler.run()`` returning the finished
requests, whose ``out_ids()`` are the new tokens (server.py:97-98, 475-479, 517-527).
``Engine`` keeps those names and adds ``generate(prompts, params)`` for the common case.
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Union

import torch

from .config.engine_config import EngineConfig
from .engine.batch import StepEntry
from .engine.runner import ModelRunner
from .engine.scheduler import PlannedEntry, PoolTooSmall, Request, Scheduler, StepPlan
from .sampling.params import SamplingParams
from .sampling.sampler import Sampler, SampleSpec
from .engine.timers import PhaseTimers

__all__ = ["Engine", "Request", "SamplingParams", "PoolTooSmall"]


#: stands in ``Request.ids`` for a token that has been drawn on the device but not read yet
PENDING = -1


@dataclass
class _InFlight:
    """A step whose tokens are still on the device."""
    requests: List[Request]
    places: List[int]                 # where in each request's ids the token will go
    device_tokens: torch.Tensor
    host_tokens: Optional[torch.Tensor]
    event: Optional[object]


class Engine:
    def __init__(self, runner: ModelRunner):
        self.runner = runner
        eng = runner.engine
        eos = getattr(runner.config, "eos_token_id", None)
        self.scheduler = Scheduler(runner.cache, max_batch=eng.max_batch, max_tokens_per_step=eng.max_tokens_per_step,
                                   max_context=runner.max_positions, admission=eng.admission, eos_token_id=eos)
        self.sampler = runner.sampler
        #: called after every model step with ([(request, position of its first token in the step,
        #: number of its tokens)], StepOutput): the way to see the step's logits (main and MTP heads)
        #: as generation goes; the step's rows wanted are the last row of every entry that is sampled
        self.step_listener = None
        self.timers = PhaseTimers(enabled=bool(eng.profile), cuda=runner.device.type == "cuda")
        #: keep one decode step in flight (see ``step``); off: every step is read back before the next
        self.pipeline = True
        self.steps_behind = 0            # steps launched before the one before them was read back
        self._inflight: Optional[_InFlight] = None
        self._host_turn = 0
        self._host_tokens = None
        if runner.device.type == "cuda":
            self._host_tokens = [torch.zeros(eng.max_batch, dtype=torch.int32).pin_memory() for _ in range(2)]

    @classmethod
    def from_folder(cls, folder: str, engine: Optional[EngineConfig] = None) -> "Engine":
        return cls(ModelRunner.from_folder(folder, engine))

    # ---- upstream's names ---------------------------------------------------------------
    def submit(self, prompt_ids: Sequence[int], params: Optional[SamplingParams] = None) -> Request:
        for t in prompt_ids:
            if not (0 <= int(t) < self.runner.vocab_size):
                raise ValueError(f"token id {t} outside the vocabulary (0..{self.runner.vocab_size - 1})")
        req = Request(prompt_ids, params)
        self.scheduler.submit(req)
        return req

    def step(self) -> List[Request]:
        """Admit what fits, run one step, sample, retire finished requests; returns those.

        While every live request is decoding and none is about to reach a limit, one step
        stays *in flight*: the next step is launched before the tokens of the one before are
        read back (they are fed to it on the device), so the GPU does not wait for the host.
        A request that ends on the end-of-sequence token is then noticed one step late; the
        extra token is dropped."""
        sch = self.scheduler
        infl = self._inflight
        if infl is not None:
            nxt = self._launch_behind(infl)
            done = self._collect(infl)
            self._inflight = nxt
            return done
        tm = self.timers
        tm.begin_step()
        with tm.host("admit"):
            for r in sch.admit():
                self.sampler.start_request(r.slot, r.params, r.ids)
        with tm.host("plan"):
            plan = sch.plan_step()
            if not plan.entries:
                return []
            entries = []
            for e in plan.entries:
                r = e.request
                spec = SampleSpec(r.params, self.sampler.request_seed(r.params, r.id), len(r.ids) - r.prompt_len) \
                    if e.sample else None
                entries.append(StepEntry(r.slot, r.ids[r.fed:r.fed + e.n_tokens],
                                         [e.n_tokens - 1] if e.sample else [], spec))
        kind = "decode" if all(e.n_tokens == 1 for e in plan.entries) else "prefill"
        with tm.host("launch"), tm.device(kind):
            out = self.runner.step(entries)
        if self.step_listener is not None:
            self.step_listener([(e.request, e.request.fed, e.n_tokens) for e in plan.entries], out)
        if self.pipeline and self._may_stay_in_flight(plan):
            self._inflight = self._defer(plan, out)
            return []
        # the step's one device-to-host read (upstream: server.py:240)
        with tm.host("read_back"):
            tokens: List[int] = out.tokens.tolist() if out.tokens is not None else []
        with tm.host("commit"):
            return sch.commit(plan, tokens)

    # ---- one step in flight -------------------------------------------------------------
    def _may_stay_in_flight(self, plan: StepPlan) -> bool:
        """Every live request gets a token from this step and none reaches a limit with it, and
        nothing waits to be admitted: the next step can be planned without the token values."""
        sch = self.scheduler
        if sch.queue or len(plan.entries) != len(sch.active):
            return False
        for e in plan.entries:
            r = e.request
            if not e.sample:
                return False
            if len(r.ids) - r.prompt_len + 1 >= r.params.max_new_tokens or len(r.ids) + 1 >= sch.max_context:
                return False
        return True

    def _defer(self, plan: StepPlan, out) -> "_InFlight":
        """Account for the step now (positions, counters) with a placeholder for each token, and
        start the copy of the drawn tokens to the host."""
        reqs, places = [], []
        for e in plan.entries:
            r = e.request
            r.fed += e.n_tokens
            places.append(len(r.ids))
            r.ids.append(PENDING)
            reqs.append(r)
        self.scheduler.steps += 1
        self.scheduler.tokens_run += plan.tokens
        host, event = None, None
        if out.tokens.is_cuda:
            host = self._host_tokens[self._host_turn]
            self._host_turn ^= 1
            host[: len(reqs)].copy_(out.tokens, non_blocking=True)
            event = torch.cuda.Event()
            event.record()
        return _InFlight(reqs, places, out.tokens, host, event)

    def _launch_behind(self, infl: "_InFlight") -> Optional["_InFlight"]:
        """Launch the step after the one in flight, if it can be planned without that one's
        tokens: same requests, one token each, pages at hand, no limit reached."""
        sch = self.scheduler
        reqs = [r for r in infl.requests if not r.done]
        if sch.queue or len(reqs) != len(sch.active) or not reqs:
            return None
        need = 0
        for r in reqs:
            if len(r.ids) - r.prompt_len + 1 >= r.params.max_new_tokens or len(r.ids) + 1 >= sch.max_context:
                return None
            need += sch.grow_pages(r, 1)
        if need > self.runner.cache.free_pages():
            return None                                  # pages are short: decide with the tokens in hand
        index = [infl.requests.index(r) for r in reqs]
        entries = [StepEntry(r.slot, [0], [0],
                             SampleSpec(r.params, self.sampler.request_seed(r.params, r.id), len(r.ids) - r.prompt_len))
                   for r in reqs]
        tm = self.timers
        tm.begin_step()
        with tm.host("launch"), tm.device("decode"):
            out = self.runner.step(entries, feed=(infl.device_tokens, index))
        if self.step_listener is not None:
            self.step_listener([(r, r.fed, 1) for r in reqs], out)
        self.steps_behind += 1
        plan = StepPlan([PlannedEntry(r, 1, True) for r in reqs])
        return self._defer(plan, out)

    def _collect(self, infl: "_InFlight") -> List[Request]:
        """Read the tokens of a step that was left in flight and finish its bookkeeping."""
        sch = self.scheduler
        with self.timers.host("read_back"):
            if infl.event is not None:
                infl.event.synchronize()
                tokens = infl.host_tokens[: len(infl.requests)].tolist()
            else:
                tokens = infl.device_tokens.tolist()
        done = []
        for r, place, tok in zip(infl.requests, infl.places, tokens):
            if r.done:
                continue                                 # ended a step earlier: this token is dropped
            r.ids[place] = int(tok)
            eos = sch.eos_token_id
            if eos is not None and not r.params.ignore_eos and tok == eos:
                del r.ids[place + 1:]                    # a placeholder of the step launched behind, if any
                r.fed = min(r.fed, len(r.ids))
                r.done, r.finish_reason = True, "eos"
                done.append(r)
        for r in done:
            sch.cache.release(r.slot)
            r.slot = None
            sch.finished.append(r)
        if done:
            sch.active = [r for r in sch.active if not r.done]
        sch.min_free_pages = min(sch.min_free_pages, sch.cache.free_pages())
        return done

    def drain(self) -> List[Request]:
        """Collect the step in flight, if any."""
        if self._inflight is None:
            return []
        infl, self._inflight = self._inflight, None
        return self._collect(infl)

    def run(self) -> List[Request]:
        """Until queue and active list are empty (upstream ``run``, server.py:475-479)."""
        while self.scheduler.has_work():
            self.step()
        self.drain()
        self.runner.check_fault()
        return self.scheduler.finished

    # ---- convenience ----------------------------------------------------------------------
    def generate(self, prompts: Sequence[Sequence[int]],
                 params: Union[None, SamplingParams, Sequence[SamplingParams]] = None) -> List[List[int]]:
        """New tokens for each prompt (lists of token ids in, lists of token ids out)."""
        if params is None or isinstance(params, SamplingParams):
            params = [params or SamplingParams()] * len(prompts)
        reqs = [self.submit(p, sp) for p, sp in zip(prompts, params)]
        self.run()
        done = {id(r) for r in reqs}
        self.scheduler.finished = [r for r in self.scheduler.finished if id(r) not in done]
        return [r.out_ids() for r in reqs]

    def stats(self) -> Dict:
        s = self.scheduler.stats()
        s.update(model_steps=self.runner.steps_run, steps_behind=self.steps_behind, rows_run=self.runner.rows_run,
                 pages=self.runner.cache.num_pages, free_pages=self.runner.cache.free_pages())
        if self.timers.enabled:
            s["phases"] = self.timers.summary()
        return s
