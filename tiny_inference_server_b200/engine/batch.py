"""What one step runs: rows (request slot, position, token) and the metadata the
kernels read.

Upstream builds, per launch, python lists turned into tensors: tokens, positions,
write pointers, a flat page table with per-row starts, kv lengths (``server.py:195-234``,
``294-318``).  Here a step is described by four int32 arrays over its rows (token,
position, slot, last row of the same request) and the device block tables of the cache
groups, which persist between steps; kernels find pages from (slot, position)
themselves.  What else a mixer's kernels want laid out per step (tiles of rows, for
instance) comes from the planners the mixers declare (``parts.base.StepPlanner``); this
module lays out whatever arrays they return and knows nothing of their meaning.  All
per-step arrays travel to the device in one copy.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch


@dataclass
class StepEntry:
    """The next tokens of one live request, and the places among them whose logits are
    wanted (indices into ``tokens``)."""
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()
    sample: object = None        # sampling.SampleSpec: draw the token after the entry's last token


@dataclass
class Segment:
    slot: int
    row0: int
    rows: int
    pos0: int


class StepContext:
    """Everything a part may know about the step.  ``positions`` and ``row_slot`` are the
    ones of the *stage* the part runs in: a stage that lags the trunk by ``lag`` positions
    sees ``position - lag`` and slot -1 (padding) where that would be negative."""

    def __init__(self, n: int, tokens, positions, row_slot, row_last, segments: List[Segment],
                 block_tables: List[torch.Tensor], page_sizes: List[int], fault: torch.Tensor,
                 max_position: int, trunk_slot=None, lag: int = 0, stages: Optional[dict] = None,
                 decode_only: bool = False, plans: Optional[Dict] = None):
        self.n = n
        self.tokens = tokens
        self.positions = positions
        self.row_slot = row_slot            # -1: padding row for this stage
        self.trunk_slot = trunk_slot if trunk_slot is not None else row_slot
        self.row_last = row_last
        self.segments = segments
        self.block_tables = block_tables
        self.page_sizes = page_sizes
        self.fault = fault
        self.max_position = max_position    # largest position among the rows (host)
        self.min_position = 0               # smallest position among the rows (host)
        self.lag = lag
        self._stages = stages if stages is not None else {}
        self.decode_only = decode_only      # every request has exactly one row
        self.want_identity = False          # the wanted rows are all rows of the step, in order (no gather needed)
        self.plans = plans if plans is not None else {}     # planner key -> what its ``bind`` returned
        self.scratch: Dict = {}             # buffers that kernels of this step may share

    def stage(self, lag: int) -> "StepContext":
        """The same rows seen by a stage that runs ``lag`` positions behind the trunk."""
        if lag == 0:
            return self
        return self._stages[lag]

    def plan(self, planner):
        """What ``planner`` (a ``parts.base.StepPlanner``) made of this step.  Planned with the
        step for the planners the model's mixers declare; for any other it is derived here from
        the device arrays (which synchronises)."""
        if planner.key not in self.plans:
            self.plans[planner.key] = planner.infer(self.stage(0).positions, self.stage(0).row_slot)
        return self.plans[planner.key]


@dataclass
class StepLayout:
    """The per-step arrays as one flat list of int32 words, and where each array lies."""
    flat: "np.ndarray"
    offsets: Dict[str, Tuple[int, int]]
    n: int
    segments: List[Segment]
    lags: List[int]
    plan_facts: Dict                 # planner key -> (index of the planner, array names, host-side facts)
    n_want: int
    max_position: int
    decode_only: bool
    min_position: int = 0
    want_identity: bool = False      # by the shape of the step, the wanted rows are all rows in order


def layout_step(entries: Sequence[StepEntry], starts: Sequence[int], lags: Sequence[int], vocab_size: int,
                pad_to: Optional[int] = None, planners: Sequence = (), want_all: bool = False,
                max_position: Optional[int] = None) -> StepLayout:
    """Lay the entries out as rows (host only, array arithmetic: no loop over tokens).
    ``starts[i]`` is the position of entry i's first token.  ``pad_to``: add padding rows
    (slot -1) up to this many rows.  ``want_all``: every row is wanted, padding included.
    ``max_position``: an upper bound to plan key splits with instead of the largest position
    of this step."""
    tok_parts, pos_parts, slot_parts, last_parts = [], [], [], []
    want_rows: List[int] = []
    segments: List[Segment] = []
    row0 = 0
    for e, start in zip(entries, starts):
        toks = np.asarray(e.tokens, dtype=np.int64)
        k = int(toks.shape[0])
        if k == 0:
            raise ValueError(f"slot {e.slot}: an entry needs at least one token")
        if toks.min() < 0 or toks.max() >= vocab_size:
            bad = int(toks[(toks < 0) | (toks >= vocab_size)][0])
            raise ValueError(f"slot {e.slot}: token id {bad} outside the vocabulary (0..{vocab_size - 1})")
        tok_parts.append(toks.astype(np.int32))
        pos_parts.append(np.arange(start, start + k, dtype=np.int32))
        slot_parts.append(np.full(k, e.slot, dtype=np.int32))
        last_parts.append(np.full(k, row0 + k - 1, dtype=np.int32))
        for w in e.want:
            if not (0 <= int(w) < k):
                raise ValueError(f"slot {e.slot}: wanted place {w} outside its {k} tokens")
            want_rows.append(row0 + int(w))
        segments.append(Segment(e.slot, row0, k, start))
        row0 += k
    n_real = row0
    n = n_real
    seg_rows = [(s.row0, s.rows) for s in segments]
    if pad_to is not None and pad_to > n:
        pad = pad_to - n
        tok_parts.append(np.zeros(pad, dtype=np.int32))
        pos_parts.append(np.zeros(pad, dtype=np.int32))
        slot_parts.append(np.full(pad, -1, dtype=np.int32))
        last_parts.append(np.arange(n, n + pad, dtype=np.int32))
        seg_rows += [(r, 1) for r in range(n, n + pad)]
        n = pad_to
    tokens = np.concatenate(tok_parts)
    positions = np.concatenate(pos_parts)
    slots = np.concatenate(slot_parts)
    last = np.concatenate(last_parts)
    lags = [l for l in sorted(set(lags)) if l > 0]
    parts: List[np.ndarray] = []
    offsets: Dict[str, Tuple[int, int]] = {}
    cursor = 0

    def put(name, values):
        nonlocal cursor
        arr = np.asarray(values, dtype=np.int32).reshape(-1)
        offsets[name] = (cursor, int(arr.shape[0]))
        parts.append(arr)
        cursor += int(arr.shape[0])

    put("tokens", tokens)
    put("positions", positions)
    put("slots", slots)
    put("last", last)
    for lag in lags:
        put(f"pos{lag}", np.maximum(positions - lag, 0))
        put(f"slot{lag}", np.where(positions - lag >= 0, slots, -1))
    facts = {}
    for i, pl in enumerate(planners):
        arrays, fact = pl.plan(seg_rows)
        facts[pl.key] = (i, tuple(arrays), fact)
        for name, values in arrays.items():
            put(f"plan{i}.{name}", values)
    if want_all:
        want_rows = list(range(n))
    put("want", want_rows)
    max_pos = int(positions[:n_real].max()) if n_real else 0
    if max_position is not None:
        max_pos = max(max_pos, max_position)
    flat = np.concatenate(parts) if parts else np.zeros(0, dtype=np.int32)
    return StepLayout(flat, offsets, n, segments, lags, facts, len(want_rows), max_pos,
                      all(s.rows == 1 for s in segments), int(positions[:n_real].min()) if n_real else 0,
                      want_identity=bool(want_all))


def layout_decode(entries: Sequence[StepEntry], starts: Sequence[int], lags: Sequence[int], vocab_size: int,
                  pad_to: int, planners: Sequence = (), max_position: Optional[int] = None) -> StepLayout:
    """``layout_step`` for the common case of a decode-only step (one token per entry, every
    row wanted, padded to ``pad_to`` rows), with plain lists: for a handful of rows that is
    several times faster than array arithmetic.  Same layout, word for word."""
    n_real = len(entries)
    n = max(pad_to, n_real)
    pad = n - n_real
    tokens = [int(e.tokens[0]) for e in entries]
    for e, t in zip(entries, tokens):
        if not (0 <= t < vocab_size):
            raise ValueError(f"slot {e.slot}: token id {t} outside the vocabulary (0..{vocab_size - 1})")
    positions = list(starts) + [0] * pad
    slots = [e.slot for e in entries] + [-1] * pad
    tokens += [0] * pad
    rows = list(range(n))
    flat: List[int] = []
    offsets: Dict[str, Tuple[int, int]] = {}

    def put(name, values):
        offsets[name] = (len(flat), len(values))
        flat.extend(values)

    put("tokens", tokens)
    put("positions", positions)
    put("slots", slots)
    put("last", rows)
    lags = [l for l in sorted(set(lags)) if l > 0]
    for lag in lags:
        put(f"pos{lag}", [p - lag if p >= lag else 0 for p in positions])
        put(f"slot{lag}", [s if p >= lag else -1 for s, p in zip(slots, positions)])
    facts = {}
    for i, pl in enumerate(planners):
        arrays, fact = pl.plan_decode(n)
        facts[pl.key] = (i, tuple(arrays), fact)
        for name, values in arrays.items():
            put(f"plan{i}.{name}", list(values))
    put("want", rows)
    max_pos = max(starts) if n_real else 0
    if max_position is not None:
        max_pos = max(max_pos, max_position)
    segments = [Segment(e.slot, i, 1, starts[i]) for i, e in enumerate(entries)]
    return StepLayout(flat, offsets, n, segments, lags, facts, n, max_pos, True, min(starts) if n_real else 0,
                      want_identity=True)


def context_from_layout(lay: StepLayout, dev: torch.Tensor, block_tables: List[torch.Tensor],
                        page_sizes: List[int], fault: torch.Tensor, planners: Sequence = ()
                        ) -> Tuple[StepContext, torch.Tensor]:
    """Views of the device copy of a layout as a StepContext; returns it and the wanted rows.
    ``planners``: the ones the layout was made with, in the same order."""

    def view(name):
        a, k = lay.offsets[name]
        return dev[a:a + k]

    plans = {}
    for pl in planners:
        i, names, fact = lay.plan_facts[pl.key]
        plans[pl.key] = pl.bind({name: view(f"plan{i}.{name}") for name in names}, fact)
    stages: Dict[int, StepContext] = {}
    ctx = StepContext(lay.n, view("tokens"), view("positions"), view("slots"), view("last"), lay.segments,
                      block_tables, page_sizes, fault, lay.max_position, stages=stages,
                      decode_only=lay.decode_only, plans=plans)
    ctx.min_position = lay.min_position
    ctx.want_identity = lay.want_identity
    for lag in lay.lags:
        st = StepContext(lay.n, view("tokens"), view(f"pos{lag}"), view(f"slot{lag}"), view("last"), lay.segments,
                         block_tables, page_sizes, fault, max(0, lay.max_position - lag), trunk_slot=view("slots"),
                         lag=lag, stages=stages, decode_only=lay.decode_only, plans=plans)
        st.scratch = ctx.scratch
        st.min_position = max(0, lay.min_position - lag)
        stages[lag] = st
    return ctx, view("want")


def build_step(entries: Sequence[StepEntry], starts: Sequence[int], lags: Sequence[int],
               block_tables: List[torch.Tensor], page_sizes: List[int], fault: torch.Tensor,
               device: torch.device, vocab_size: int, pad_to: Optional[int] = None,
               planners: Sequence = ()) -> Tuple[StepContext, torch.Tensor, int]:
    """Rows, metadata and context of one step; all per-step arrays go to the device in one
    copy.  Returns the context, the device indices of the wanted rows, and their count."""
    lay = layout_step(entries, starts, lags, vocab_size, pad_to=pad_to, planners=planners)
    dev = torch.from_numpy(lay.flat).to(device, non_blocking=True)
    ctx, want = context_from_layout(lay, dev, block_tables, page_sizes, fault, planners)
    return ctx, want, lay.n_want


class StaticMeta:
    """A fixed device buffer for the per-step arrays of steps that all have the same layout
    (the same number of rows, tiles and wanted rows), filled through a small ring of pinned
    host buffers: a host buffer is written again only after the copy that read it last has
    finished, so the host may run ahead of the device."""

    RING = 4

    def __init__(self, capacity: int, device: torch.device):
        cuda = device.type == "cuda"
        self.hosts = [torch.zeros(capacity, dtype=torch.int32).pin_memory() if cuda else
                      torch.zeros(capacity, dtype=torch.int32) for _ in range(self.RING)]
        self.events = [torch.cuda.Event() if cuda else None for _ in range(self.RING)]
        self.recorded = [False] * self.RING
        self.turn = 0
        self.dev = torch.zeros(capacity, dtype=torch.int32, device=device)
        self.layout: Optional[Dict[str, Tuple[int, int]]] = None
        self.used = 0

    def upload(self, flat, offsets: Dict[str, Tuple[int, int]]) -> torch.Tensor:
        if len(flat) > self.dev.numel():
            raise ValueError(f"step metadata of {len(flat)} words exceeds the static buffer ({self.dev.numel()})")
        if self.layout is None:
            self.layout = dict(offsets)
            self.used = len(flat)
        elif self.layout != offsets:
            raise ValueError("the layout of a step's metadata changed under a captured graph")
        i = self.turn
        self.turn = (self.turn + 1) % self.RING
        if self.recorded[i]:
            self.events[i].synchronize()
        host = self.hosts[i]
        host[: self.used] = torch.from_numpy(flat) if isinstance(flat, np.ndarray) else \
            torch.tensor(flat, dtype=torch.int32)
        self.dev[: self.used].copy_(host[: self.used], non_blocking=True)
        if self.events[i] is not None:
            self.events[i].record()
            self.recorded[i] = True
        return self.dev
