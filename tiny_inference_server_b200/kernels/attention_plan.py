"""How the tensor-core attention kernels (csrc/attention_mma.cu, csrc/attention_tc.cu) want the
rows of a step cut into tiles, and the planner that tells the engine so.

The tile geometry belongs to the kernels: a CTA of the mma.sync kernel takes the G query heads of
one kv head for up to 16 // G rows when it splits the keys (decode rows, tiny portions), or up to
64 // G rows of a prompt portion; the tcgen05 kernel takes up to 128 rows of one query head.  The
engine knows none of this: a mixer hands it a planner (``Mixer.step_planners``), the engine calls
the planner with the step's segments while it lays the step out on the host, uploads the arrays
the planner returns together with the step's own, and gives the planner the device views back.
"""
from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

import torch

from ..parts.base import StepPlanner

#: rows from which a portion of a prompt is also cut into wide tiles (for the tcgen05 kernel)
WIDE_MIN_ROWS = 64
WIDE_TILE_ROWS = 128


class TileSet:
    """Attention work of one step for one group size G (query heads per kv head): tiles of
    consecutive rows of one request.  ``keys``: tiles of at most 16 // G rows (decode rows,
    tiny portions), whose keys are split over warps and CTAs; ``rows``: tiles of at most
    64 // G rows (portions of prompts).  Each is (first rows, row counts, number of tiles);
    the first two are int32 device tensors.  ``wide``: the portions of at least WIDE_MIN_ROWS
    rows once more, as tiles of up to 128 rows, for the kernel that takes those; their ``rows``
    tiles are the first ``rows_in_wide`` of ``rows``, so a caller runs either ``wide`` and the
    rest of ``rows``, or all of ``rows``."""

    def __init__(self, keys, rows, keys_max_rows: int = 0, wide=None, rows_in_wide: int = 0, keys_identity: bool = False):
        self.keys = keys
        self.rows = rows
        self.keys_max_rows = keys_max_rows      # the most rows of any ``keys`` tile (0: not known)
        self.keys_identity = keys_identity      # ``keys`` tile i is row i alone (a decode step): a kernel need not read the arrays
        self.wide = wide if wide is not None else (None, None, 0)
        self.rows_in_wide = rows_in_wide


def plan_tiles(segments: Sequence[Tuple[int, int]], group_size: int):
    """Cut (row0, rows) segments into tiles.  Returns (keys tiles, rows tiles, wide tiles, number
    of leading rows tiles that the wide tiles cover) with tiles as lists of (row0, rows)."""
    r_keys = 16 // group_size if group_size <= 16 else 0
    r_rows = max(1, 64 // group_size)
    keys, rows_wide, rows_rest, wide = [], [], [], []
    for row0, n in segments:
        if r_keys and n <= r_keys:
            keys.append((row0, n))
            continue
        into = rows_rest
        if n >= WIDE_MIN_ROWS:
            into = rows_wide
            for a in range(0, n, WIDE_TILE_ROWS):
                wide.append((row0 + a, min(WIDE_TILE_ROWS, n - a)))
        for a in range(0, n, r_rows):
            into.append((row0 + a, min(r_rows, n - a)))
    return keys, rows_wide + rows_rest, wide, len(rows_wide)


class AttentionTilePlanner(StepPlanner):
    """Tiles for mixers with ``group_size`` query heads per kv head (``TileSet``)."""

    ARRAYS = ("k0", "kn", "r0", "rn", "w0", "wn")

    def __init__(self, group_size: int):
        self.group_size = group_size
        self.key = ("attention_tiles", group_size)

    def max_words(self, rows: int) -> int:
        # every row is in one keys tile or one rows tile, and at most once more in a wide tile
        return 4 * rows

    def plan(self, segments: Sequence[Tuple[int, int]]):
        keys, rows, wide, rows_in_wide = plan_tiles(segments, self.group_size)
        arrays = {"k0": [t[0] for t in keys], "kn": [t[1] for t in keys],
                  "r0": [t[0] for t in rows], "rn": [t[1] for t in rows],
                  "w0": [t[0] for t in wide], "wn": [t[1] for t in wide]}
        # (the last fact: the keys tiles are the step's rows, one each and in order, and there are no others)
        identity = bool(keys) and not rows and not wide and all(t == (i, 1) for i, t in enumerate(keys))
        facts = (len(keys), len(rows), max((t[1] for t in keys), default=0), len(wide), rows_in_wide, identity)
        return arrays, facts

    def plan_decode(self, rows: int):
        idx, ones = list(range(rows)), [1] * rows
        if self.group_size <= 16:
            return {"k0": idx, "kn": ones, "r0": [], "rn": [], "w0": [], "wn": []}, (rows, 0, 1, 0, 0, True)
        return {"k0": [], "kn": [], "r0": idx, "rn": ones, "w0": [], "wn": []}, (0, rows, 0, 0, 0, False)

    def bind(self, arrays: Dict[str, torch.Tensor], facts) -> TileSet:
        nk, nr, kmax, nw, nrw = facts[:5]
        return TileSet((arrays["k0"], arrays["kn"], nk), (arrays["r0"], arrays["rn"], nr), kmax,
                       (arrays["w0"], arrays["wn"], nw), nrw, keys_identity=len(facts) > 5 and bool(facts[5]))


_planners: Dict[int, AttentionTilePlanner] = {}


def planner(group_size: int) -> AttentionTilePlanner:
    p = _planners.get(group_size)
    if p is None:
        p = _planners[group_size] = AttentionTilePlanner(group_size)
    return p


def infer_tiles(positions: torch.Tensor, row_slot: torch.Tensor, group_size: int) -> TileSet:
    """Tiles from the device arrays alone (synchronises; for calls outside a step, as in kernel
    tests)."""
    return planner(group_size).infer(positions, row_slot)
