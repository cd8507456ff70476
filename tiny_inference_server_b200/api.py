"""The Python entry point: ``Engine`` — submit requests, step, run, ``generate``.

Upstream's entry is ``Scheduler.submit`` + ``Scheduler.run()`` returning the finished
requests, whose ``out_ids()`` are the new tokens (server.py:97-98, 475-479, 517-527).
``Engine`` keeps those names and adds ``generate(prompts, params)`` for the common case.
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional, Sequence, Union

import torch

from .config.engine_config import EngineConfig
from .engine.batch import StepEntry
from .engine.runner import ModelRunner
from .engine.scheduler import PoolTooSmall, Request, Scheduler, StepPlan
from .sampling.params import SamplingParams
from .sampling.sampler import Sampler, SampleSpec

__all__ = ["Engine", "Request", "SamplingParams", "PoolTooSmall"]


class Engine:
    def __init__(self, runner: ModelRunner):
        self.runner = runner
        eng = runner.engine
        eos = getattr(runner.config, "eos_token_id", None)
        self.scheduler = Scheduler(runner.cache, max_batch=eng.max_batch, max_tokens_per_step=eng.max_tokens_per_step,
                                   max_context=runner.max_positions, admission=eng.admission, eos_token_id=eos)
        self.sampler = runner.sampler
        self.last_aux = None

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
        """Admit what fits, run one step, sample, retire finished requests; returns those."""
        sch = self.scheduler
        for r in sch.admit():
            self.sampler.start_request(r.slot, r.params, r.ids)
        plan = sch.plan_step()
        if not plan.entries:
            return []
        entries = []
        for e in plan.entries:
            r = e.request
            spec = SampleSpec(r.params, self.sampler.request_seed(r.params, r.id), len(r.ids) - r.prompt_len) \
                if e.sample else None
            entries.append(StepEntry(r.slot, r.ids[r.fed:r.fed + e.n_tokens], [e.n_tokens - 1] if e.sample else [],
                                     spec))
        out = self.runner.step(entries)
        self.last_aux = out.aux
        # the step's one device-to-host read (upstream: server.py:240)
        tokens: List[int] = out.tokens.tolist() if out.tokens is not None else []
        return sch.commit(plan, tokens)

    def run(self) -> List[Request]:
        """Until queue and active list are empty (upstream ``run``, server.py:475-479)."""
        while self.scheduler.has_work():
            self.step()
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
        s.update(model_steps=self.runner.steps_run, rows_run=self.runner.rows_run,
                 pages=self.runner.cache.num_pages, free_pages=self.runner.cache.free_pages())
        return s
