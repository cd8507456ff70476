"""The step function: model + cache manager + one ``step``.

``step`` takes a batch of (request slot, its next tokens) — portions of prompts beside
single decoded tokens, cut anywhere — runs exactly those tokens as one batch against
the cache that earlier steps left, and returns the logits at the wanted places.
Upstream has two launch paths that are never mixed in one launch (whole prompts from an
empty cache, ``prefill_rows``; rows over the paged cache, ``trunk_rows``:
main_models_new.py:197-217, server.py:279-284); here there is one.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from ..cache.manager import CacheManager
from ..cache.pages import CacheError, OutOfPages
from ..config.engine_config import EngineConfig
from ..kernels import ops
from ..models.base import Model, StepOutput
from ..parts.base import BuildContext
from ..registry import build_model, config_from_folder
from ..weights.loader import check_tensors, load_weights
from .batch import StepEntry, build_step

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


class DeviceFault(RuntimeError):
    """A kernel met a page id outside its pool (the block tables and the batch disagree)."""


def feed_tokens(dst: torch.Tensor, n: int, feed) -> None:
    """dst[i] = tokens[index[i]] for the first ``n`` rows, on the device (stream-ordered)."""
    src, index = feed
    if list(index) == list(range(n)):
        dst[:n].copy_(src[:n])
    else:
        dst[:n].copy_(src.index_select(0, torch.tensor(list(index), dtype=torch.int64, device=src.device)))


class ModelRunner:
    def __init__(self, cfg, tensors: Dict[str, torch.Tensor], engine: Optional[EngineConfig] = None):
        self.engine = engine or EngineConfig()
        self.config = cfg
        self.device = torch.device(self.engine.device)
        self.dtype = _DTYPES[self.engine.dtype]
        self.build_ctx = BuildContext(self.device, self.dtype)
        self.model: Model = build_model(cfg)
        check_tensors(tensors, self.model.expected_tensors())
        self.model.load(tensors, self.build_ctx)
        self.vocab_size = self.model.vocab_size
        self.max_positions = min(self.model.max_positions, self.engine.max_context or self.model.max_positions)
        kv_specs = self.model.kv_specs()
        elem = torch.empty((), dtype=self.dtype).element_size()
        page_bytes = CacheManager.bytes_per_page(kv_specs, self.engine.page_size, elem)
        num_pages = self.engine.num_pages
        if num_pages is None:
            num_pages = max(1, self.engine.pool_bytes // max(1, page_bytes))
        self.cache = CacheManager(kv_specs, self.model.state_specs(self.build_ctx), page_size=self.engine.page_size,
                                  num_pages=num_pages, max_slots=self.engine.max_batch,
                                  max_positions=self.max_positions, dtype=self.dtype, device=self.device,
                                  debug_poison=self.engine.debug_poison)
        self.model.bind(self.cache)
        self.fault = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.lags = self.model.lags()
        # what the mixers' kernels want planned with every step; one planner per key
        self.planners = []
        for p in self.model.walk_parts():
            for pl in (p.step_planners() if hasattr(p, "step_planners") else ()):
                if all(pl.key != q.key for q in self.planners):
                    self.planners.append(pl)
        self.aux = bool(self.engine.mtp)
        from ..sampling.sampler import Sampler
        self.sampler = Sampler(self.vocab_size, self.engine.max_batch, self.device, seed=self.engine.seed)
        self.graphs = None
        self.step_graphs = None
        if self.engine.cuda_graphs and self.device.type == "cuda" and all(p.graph_safe for p in self.model.walk_parts()):
            from .graphs import DecodeGraphs, StepGraphs
            self.graphs = DecodeGraphs(self)
            self.step_graphs = StepGraphs(self)
        self.steps_run = 0
        self.rows_run = 0

    @classmethod
    def from_folder(cls, folder: str, engine: Optional[EngineConfig] = None) -> "ModelRunner":
        cfg = config_from_folder(folder)
        model = build_model(cfg)
        tensors = load_weights(folder, model.expected_tensors())
        return cls(cfg, tensors, engine)

    # ---- requests ---------------------------------------------------------------------
    def add_request(self) -> int:
        return self.cache.admit()

    def release(self, slot: int) -> None:
        self.cache.release(slot)

    def length(self, slot: int) -> int:
        return self.cache.length[slot]

    # ---- the step ---------------------------------------------------------------------
    def step(self, entries: Sequence[StepEntry], pad_to: Optional[int] = None, feed=None) -> StepOutput:
        """Run one step.  ``feed = (tokens, index)``: the step holds one token per entry and entry
        i's token is not in ``entries`` (a placeholder stands there) but on the device, at
        ``tokens[index[i]]`` — the tokens the step before drew, which the host has not read yet."""
        if not entries:
            raise ValueError("a step needs at least one entry")
        slots = [e.slot for e in entries]
        if len(set(slots)) != len(slots):
            raise ValueError("a request appears twice in one step")
        # pages and context: either every entry fits or nothing is changed
        lengths = self.cache.length
        for e in entries:
            if lengths[e.slot] + len(e.tokens) > self.max_positions:
                raise CacheError(f"slot {e.slot}: {lengths[e.slot] + len(e.tokens)} tokens exceed "
                                 f"the context limit {self.max_positions}")
        for grp in self.cache.groups:
            need = 0
            windowed = grp.window is not None
            for e in entries:
                start = lengths[e.slot]
                need += grp.pages_to_grow(e.slot, start + len(e.tokens))
                if windowed:
                    need -= grp.pages_freed_by(e.slot, start)
            if need > grp.pool.free:
                raise OutOfPages(f"group {grp.gid}: the step needs {need} pages, {grp.pool.free} are free")
        starts = [self.cache.extend(e.slot, len(e.tokens)) for e in entries]
        self.cache.sync_tables()
        if self.graphs is not None and pad_to is None and all(len(e.tokens) == 1 for e in entries):
            self.steps_run += 1
            self.rows_run += len(entries)
            return self.graphs.step(entries, starts, feed)
        if self.step_graphs is not None and pad_to is None and feed is None and sum(len(e.tokens) for e in entries) >= 64:
            out = self.step_graphs.step(entries, starts)
            if out is not None:
                self._sample(entries, out)
                self.steps_run += 1
                self.rows_run += sum(len(e.tokens) for e in entries)
                return out
        ctx, want_rows, _ = build_step(entries, starts, self.lags,
                                       [g.table_dev for g in self.cache.groups],
                                       [g.page_size for g in self.cache.groups], self.fault, self.device,
                                       self.vocab_size, pad_to=pad_to, planners=self.planners)
        if feed is not None:
            feed_tokens(ctx.tokens, len(entries), feed)
        out = self.model.forward(ctx, want_rows, aux=self.aux)
        self._sample(entries, out)
        self.steps_run += 1
        self.rows_run += ctx.n
        return out

    def _sample(self, entries: Sequence[StepEntry], out: StepOutput) -> None:
        """Draw a token for every entry that asks for one (its last wanted row)."""
        rows, specs, slots = [], [], []
        k = 0
        for e in entries:
            if e.sample is not None:
                if not len(e.want):
                    raise ValueError(f"slot {e.slot}: an entry that wants a sample must want a row's logits")
                rows.append(k + len(e.want) - 1)
                specs.append(e.sample)
                slots.append(e.slot)
            k += len(e.want)
        if not rows:
            return
        logits = out.main if rows == list(range(out.main.shape[0])) else \
            out.main.index_select(0, torch.tensor(rows, dtype=torch.int64, device=self.device))
        out.tokens = self.sampler.sample_specs(logits, specs, slots)

    def check_fault(self) -> None:
        """Synchronises.  Raises if a kernel saw a page id outside its pool."""
        code = int(self.fault[0].item())
        if code:
            self.fault.zero_()
            raise DeviceFault(f"a kernel met an invalid page id (code {code})")
        if self.device.type == "cuda" and ops._tc_fault is not None and int(ops._tc_fault[0].item()):
            ops._tc_fault.zero_()
            raise DeviceFault("a wait inside a tcgen05 matrix product ran out")
