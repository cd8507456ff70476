"""Decode-only steps replayed from CUDA graphs.

A decode step launches the same kernels with the same arguments whatever requests it
holds: what changes (tokens, positions, slots, tiles) lies in one fixed device buffer,
and the block tables are fixed device tensors.  So the step is captured once per
(number of rows rounded up to a power of two, bound on the context length) and replayed
afterwards: one launch instead of hundreds (upstream's own first item of future work:
"roughly 1000 small kernel launches" per iteration keep its GPU ~7 % busy).

Rows beyond the live requests are padding (slot -1): they write nothing into the cache
and their logits are not returned.  Logits are computed for every row of the bucket.
"""
from __future__ import annotations

import gc
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..kernels import ops
from ..models.base import StepOutput
from ..sampling.sampler import WORDS_PER_ROW
from .batch import StaticMeta, StepEntry, context_from_layout, layout_decode, layout_step


def _next_pow2(x: int) -> int:
    return 1 << max(0, (x - 1).bit_length())


class GraphedDecode:
    """One captured decode step for ``bucket`` rows and contexts up to ``kv_bound`` keys."""

    def __init__(self, runner, bucket: int, kv_bound: int, sampled: bool):
        self.runner = runner
        self.bucket = bucket
        self.kv_bound = kv_bound
        self.sampled = sampled            # the graph also draws a token for every row
        # tokens, positions, slots, last row; two arrays per lagging stage; the planners' arrays; wanted rows
        words = (4 + 2 * len([l for l in runner.lags if l > 0]) + 1 + WORDS_PER_ROW) * bucket
        words += sum(pl.max_words(bucket) for pl in runner.planners)
        self.static = StaticMeta(words + 16, runner.device)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.out: Optional[StepOutput] = None
        self.kernels = 0                # launches of this library's kernels inside the graph

    def run(self, entries: Sequence[StepEntry], starts: Sequence[int], feed=None) -> StepOutput:
        r = self.runner
        lay = layout_decode(entries, starts, r.lags, r.vocab_size, self.bucket, r.planners,
                            max_position=self.kv_bound - 1)
        if self.sampled:
            if len(lay.flat) % 2:
                lay.flat.append(0)        # the block of sampling parameters starts 8-byte aligned
            lay.offsets["sampling"] = (len(lay.flat), WORDS_PER_ROW * self.bucket)
            lay.flat.extend(r.sampler.pack([e.sample for e in entries], [e.slot for e in entries], self.bucket))
        dev = self.static.upload(lay.flat, lay.offsets)
        if feed is not None:
            from .runner import feed_tokens
            a, _ = lay.offsets["tokens"]
            feed_tokens(dev[a:a + len(entries)], len(entries), feed)
        if self.graph is not None:
            self.graph.replay()
            ops.launches += self.kernels
            return self.out
        # first time: run the step as it is (this is the real step), then capture it
        tables = [g.table_dev for g in r.cache.groups]
        sizes = [g.page_size for g in r.cache.groups]
        ctx, want = context_from_layout(lay, dev, tables, sizes, r.fault, r.planners)
        words = None
        if self.sampled:
            a, k = lay.offsets["sampling"]
            words = dev[a:a + k]

        def run_once() -> StepOutput:
            o = r.model.forward(ctx, want, aux=r.aux)
            if words is not None:
                o.tokens = r.sampler.sample_packed(o.main, words)
            return o

        out = run_once()
        torch.cuda.synchronize(r.device)
        before = ops.launches
        graph, self.out = _capture(run_once)
        self.kernels = ops.launches - before
        ops.launches = before           # captured, not run
        self.graph = graph
        return out


class DecodeGraphs:
    def __init__(self, runner, min_kv: int = 512):
        self.runner = runner
        self.min_kv = min_kv
        self.graphs: Dict[Tuple[int, int], GraphedDecode] = {}
        self.replays = 0

    def step(self, entries: Sequence[StepEntry], starts: Sequence[int], feed=None) -> StepOutput:
        r = self.runner
        n = len(entries)
        bucket = min(_next_pow2(n), max(n, r.engine.max_batch))
        max_kv = max(starts) + 1
        kv_bound = min(max(self.min_kv, _next_pow2(max_kv)), max(r.max_positions, max_kv))
        sampled = any(e.sample is not None for e in entries)
        key = (bucket, kv_bound, sampled)
        g = self.graphs.get(key)
        if g is None:
            g = self.graphs[key] = GraphedDecode(r, bucket, kv_bound, sampled)
        else:
            self.replays += 1
        full = g.run(entries, starts, feed)
        wanted = [i for i, e in enumerate(entries) if len(e.want)]
        drawn = [i for i, e in enumerate(entries) if e.sample is not None]
        tokens = None
        if full.tokens is not None and drawn:
            tokens = full.tokens[: len(drawn)] if drawn == list(range(len(drawn))) else \
                full.tokens.index_select(0, torch.tensor(drawn, dtype=torch.int64, device=r.device))
        if wanted == list(range(len(wanted))):
            k = len(wanted)
            return StepOutput(main=full.main[:k], aux=[a[:k] for a in full.aux],
                              aux_valid=[v[:k] for v in full.aux_valid], tokens=tokens)
        idx = torch.tensor(wanted, dtype=torch.int64, device=r.device)
        return StepOutput(main=full.main.index_select(0, idx), aux=[a.index_select(0, idx) for a in full.aux],
                          aux_valid=[v.index_select(0, idx) for v in full.aux_valid], tokens=tokens)


def _capture(run_once):
    """Capture ``run_once`` into a CUDA graph; returns (graph, what run_once returned)."""
    graph = torch.cuda.CUDAGraph()
    # No garbage collection while the stream is capturing: the collector may destroy an
    # older engine's graphs, and destroying a graph invalidates a capture in progress.
    gc.collect()
    was_enabled = gc.isenabled()
    gc.disable()
    try:
        with torch.cuda.graph(graph):
            out = run_once()
    finally:
        if was_enabled:
            gc.enable()
    return graph, out


class GraphedStep:
    """One captured step of a fixed shape: the same number of entries with the same numbers of
    tokens and the same wanted places, contexts up to ``kv_bound`` keys."""

    def __init__(self, runner, kv_bound: int):
        self.runner = runner
        self.kv_bound = kv_bound
        self.static: Optional[StaticMeta] = None
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.out: Optional[StepOutput] = None
        self.kernels = 0

    def run(self, entries: Sequence[StepEntry], starts: Sequence[int]) -> StepOutput:
        r = self.runner
        lay = layout_step(entries, starts, r.lags, r.vocab_size, planners=r.planners,
                          max_position=self.kv_bound - 1)
        if self.static is None:
            self.static = StaticMeta(len(lay.flat) + 16, r.device)
        dev = self.static.upload(lay.flat, lay.offsets)
        if self.graph is not None:
            self.graph.replay()
            ops.launches += self.kernels
            return self.out
        # first time: run the step as it is (this is the real step), then capture it
        lay.min_position = 0            # planned for any positions up to the bound, not for this step's
        ctx, want = context_from_layout(lay, dev, [g.table_dev for g in r.cache.groups],
                                        [g.page_size for g in r.cache.groups], r.fault, r.planners)

        def run_once() -> StepOutput:
            return r.model.forward(ctx, want, aux=r.aux)

        out = run_once()
        torch.cuda.synchronize(r.device)
        before = ops.launches
        self.graph, self.out = _capture(run_once)
        self.kernels = ops.launches - before
        ops.launches = before           # captured, not run
        return out


class StepGraphs:
    """Graphs for steps other than decode-only ones (portions of prompts, mixed steps) whose shape
    comes back: a server that cuts prompts into portions of its token budget runs the same shape
    again and again.  A shape is captured when it is seen for the second time; the least recently
    used graphs beyond ``capacity`` are dropped (each holds the step's activations)."""

    def __init__(self, runner, capacity: int = 6, min_kv: int = 512):
        self.runner = runner
        self.capacity = capacity
        self.min_kv = min_kv
        self.seen: Dict[tuple, int] = {}
        self.graphs: Dict[tuple, GraphedStep] = {}
        self.replays = 0

    def key(self, entries: Sequence[StepEntry], starts: Sequence[int]) -> tuple:
        r = self.runner
        max_kv = max(s + len(e.tokens) for e, s in zip(entries, starts))
        kv_bound = min(max(self.min_kv, _next_pow2(max_kv)), max(r.max_positions, max_kv))
        return (kv_bound,) + tuple((len(e.tokens), tuple(e.want)) for e in entries)

    def step(self, entries: Sequence[StepEntry], starts: Sequence[int]) -> Optional[StepOutput]:
        """The step's output from a graph, or None: the caller runs the step eagerly."""
        key = self.key(entries, starts)
        g = self.graphs.get(key)
        if g is None:
            n = self.seen.get(key, 0) + 1
            self.seen[key] = n
            if len(self.seen) > 4096:
                self.seen.clear()
            if n < 2:
                return None
            while len(self.graphs) >= self.capacity:
                self.graphs.pop(next(iter(self.graphs)))
            g = GraphedStep(self.runner, key[0])
        else:
            self.graphs.pop(key)        # re-inserted below: most recently used last
            self.replays += 1
        self.graphs[key] = g
        return g.run(entries, starts)
