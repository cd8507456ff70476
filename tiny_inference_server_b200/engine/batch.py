"""What one step runs: rows (request slot, position, token) and the metadata the
kernels read.

Upstream builds, per launch, python lists turned into tensors: tokens, positions,
write pointers, a flat page table with per-row starts, kv lengths (``server.py:195-234``,
``294-318``).  Here a step is described by four int32 arrays over its rows (token,
position, slot, last row of the same request) and the device block tables of the cache
groups, which persist between steps; kernels find pages from (slot, position)
themselves.  All per-step arrays travel to the device in one copy.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch


@dataclass
class StepEntry:
    """The next tokens of one live request, and the places among them whose logits are
    wanted (indices into ``tokens``)."""
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


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
                 decode_only: bool = False):
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
        self.lag = lag
        self._stages = stages if stages is not None else {}
        self.decode_only = decode_only      # every request has exactly one row

    def stage(self, lag: int) -> "StepContext":
        """The same rows seen by a stage that runs ``lag`` positions behind the trunk."""
        if lag == 0:
            return self
        return self._stages[lag]


def build_step(entries: Sequence[StepEntry], starts: Sequence[int], lags: Sequence[int],
               block_tables: List[torch.Tensor], page_sizes: List[int], fault: torch.Tensor,
               device: torch.device, vocab_size: int, pad_to: Optional[int] = None
               ) -> Tuple[StepContext, torch.Tensor, int]:
    """Lay the entries out as rows.  ``starts[i]`` is the position of entry i's first token.
    Returns the context, the device indices of the wanted rows, and their count."""
    tokens: List[int] = []
    positions: List[int] = []
    slots: List[int] = []
    last: List[int] = []
    want_rows: List[int] = []
    segments: List[Segment] = []
    for e, start in zip(entries, starts):
        k = len(e.tokens)
        if k == 0:
            raise ValueError(f"slot {e.slot}: an entry needs at least one token")
        row0 = len(tokens)
        for t in e.tokens:
            if not (0 <= int(t) < vocab_size):
                raise ValueError(f"slot {e.slot}: token id {t} outside the vocabulary (0..{vocab_size - 1})")
        tokens += [int(t) for t in e.tokens]
        positions += list(range(start, start + k))
        slots += [e.slot] * k
        last += [row0 + k - 1] * k
        for w in e.want:
            if not (0 <= int(w) < k):
                raise ValueError(f"slot {e.slot}: wanted place {w} outside its {k} tokens")
            want_rows.append(row0 + int(w))
        segments.append(Segment(e.slot, row0, k, start))
    n_real = len(tokens)
    n = n_real
    if pad_to is not None and pad_to > n:
        pad = pad_to - n
        tokens += [0] * pad
        positions += [0] * pad
        slots += [-1] * pad
        last += list(range(n, n + pad))
        n = pad_to
    lags = [l for l in sorted(set(lags)) if l > 0]
    rows = [tokens, positions, slots, last]
    for lag in lags:
        rows.append([max(0, p - lag) for p in positions])
        rows.append([s if p - lag >= 0 else -1 for s, p in zip(slots, positions)])
    packed = torch.tensor(rows, dtype=torch.int32)
    dev = packed.to(device, non_blocking=True)
    want_dev = torch.tensor(want_rows, dtype=torch.int64).to(device, non_blocking=True)
    max_pos = max(positions[:n_real]) if n_real else 0
    decode_only = all(s.rows == 1 for s in segments)
    stages: Dict[int, StepContext] = {}
    ctx = StepContext(n, dev[0], dev[1], dev[2], dev[3], segments, block_tables, page_sizes, fault, max_pos,
                      stages=stages, decode_only=decode_only)
    for i, lag in enumerate(lags):
        stages[lag] = StepContext(n, dev[0], dev[4 + 2 * i], dev[5 + 2 * i], dev[3], segments, block_tables,
                                  page_sizes, fault, max(0, max_pos - lag), trunk_slot=dev[2], lag=lag,
                                  stages=stages, decode_only=decode_only)
    return ctx, want_dev, len(want_rows)
