"""Pages of keys and values.

Upstream keeps one pool tensor for all layers, a deque of free page ids and a python
list of page ids per request (``block_table.py:31-86``).  Here the planes (one per
cached layer) are first grouped by what they need — kv heads, the widths of a key and of a
value row, and whether they keep every key or a window of them — and every group has pages of its own: a pool
tensor ``[planes, pages, 2, kv_heads, page_size, head_dim]``, a free list, and one
block table per request slot.  A page id addresses the same page in every plane of its
group, as upstream's does in every layer.

Row format.  Inside a page the keys (and the values) of one kv head are ``page_size`` rows
of ``head_dim`` elements.  Each row is stored as 16-byte chunks *permuted by the token's
position* (``cache_chunk`` in ``csrc/common.cuh``): rows of a multiple of eight chunks keep
logical chunk ``c`` at chunk ``c XOR (position mod 8)`` — the 128-byte swizzle of the
tensor-core operand layouts, applied in memory — other rows at chunk
``(c + position) mod chunks_per_row``.  The attention kernels copy a page's rows into shared
memory unchanged, in bulk copies, and the permutation is what lets them read the dense rows
there without bank conflicts, or hand them to the tensor cores as they are.  Only kernels
read and write the pages; anything else that does (tests) has to apply the same permutation.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from ..parts.base import KVSpec


class CacheError(RuntimeError):
    """Misuse of the cache manager (double free, unknown slot, pool exhausted)."""


class OutOfPages(CacheError):
    """A group has fewer free pages than an extension needs.  Nothing was allocated."""


class PagePool:
    """Free list over page ids 0..num_pages-1 (FIFO, as upstream's deque:
    ``block_table.py:44,57-63``), with the checks upstream does not make: a page is never
    handed out twice, freed twice, or freed without having been handed out."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise CacheError(f"a pool needs at least one page, got {num_pages}")
        self.num_pages = num_pages
        self._free = deque(range(num_pages))
        self._held = [False] * num_pages
        self.allocations = 0          # pages handed out so far (more than num_pages: pages were used again)

    @property
    def free(self) -> int:
        return len(self._free)

    def allocate(self) -> int:
        if not self._free:
            raise OutOfPages("no free page")
        p = self._free.popleft()
        if self._held[p]:
            raise CacheError(f"page {p} was on the free list while held")
        self._held[p] = True
        self.allocations += 1
        return p

    def release(self, page: int) -> None:
        if not (0 <= page < self.num_pages):
            raise CacheError(f"page id {page} is outside the pool (0..{self.num_pages - 1})")
        if not self._held[page]:
            raise CacheError(f"page {page} freed twice (or never allocated)")
        self._held[page] = False
        self._free.append(page)

    def shuffle(self, rng) -> None:
        """Scatter the free list (tests: pages of a request are not contiguous)."""
        items = list(self._free)
        rng.shuffle(items)
        self._free = deque(items)

    def check(self) -> None:
        """Every page is either held or exactly once on the free list."""
        on_list = [0] * self.num_pages
        for p in self._free:
            on_list[p] += 1
        for p in range(self.num_pages):
            if on_list[p] + (1 if self._held[p] else 0) != 1:
                raise CacheError(f"page {p}: on free list {on_list[p]} times, held={self._held[p]}")


@dataclass
class PlaneRef:
    """Where the cache of one schedule entry lives."""
    group: int
    index: int        # plane inside the group's pool


#: What a page is filled with when it is given back in the debugging mode: 2^100, large and finite.
#: The attention kernels may multiply a masked key's probability (exactly 0) with whatever the page
#: holds there, so the pattern must not be NaN or infinite; but a key read in earnest from a page that
#: its request no longer holds — one key too many, a stale block-table entry — now gives a score of
#: the order of 1e30, and the logits show it, instead of a drift in the third digit.
POISON = 2.0 ** 100


class CacheGroup:
    """Planes with the same needs: one pool of pages, one block table per slot."""

    def __init__(self, gid: int, kv_heads: int, head_dim: int, window: Optional[int], lags: Sequence[int],
                 page_size: int, num_pages: int, max_slots: int, max_positions: int, dtype: torch.dtype,
                 device: torch.device, v_dim: Optional[int] = None, poison: bool = False):
        self.gid = gid
        self.poison = poison                      # fill pages with POISON when they are given back
        self.kv_heads = kv_heads
        self.head_dim = head_dim                  # elements of a key row
        self.v_dim = head_dim if v_dim is None else v_dim      # elements of a value row
        self.window = window
        self.lags = list(lags)                    # per plane: how far it is filled behind the trunk
        self.max_lag = max(self.lags) if self.lags else 0
        self.page_size = page_size
        self.num_planes = len(self.lags)
        self.pool = PagePool(num_pages)
        self.max_pages_per_slot = (max_positions + page_size - 1) // page_size
        # zeros, not empty: an unwritten tail of a page must not hold NaN patterns
        # (upstream's reason too, block_table.py:40-41)
        # A page is its key rows [kv_heads, page_size, k_dim] followed by its value rows
        # [kv_heads, page_size, v_dim]; with keys and values of one width that is the 5-D shape below.
        if self.v_dim == head_dim:
            self.pages = torch.zeros((self.num_planes, num_pages, 2, kv_heads, page_size, head_dim),
                                     dtype=dtype, device=device)
        else:
            self.pages = torch.zeros((self.num_planes, num_pages, kv_heads * page_size * (head_dim + self.v_dim)),
                                     dtype=dtype, device=device)
        self.table_host = torch.full((max_slots, self.max_pages_per_slot), -1, dtype=torch.int32)
        self.table_dev = torch.full((max_slots, self.max_pages_per_slot), -1, dtype=torch.int32, device=device)
        # per slot: first logical page still held, and one past the last
        self.first = [0] * max_slots
        self.end = [0] * max_slots
        self.pending: List[tuple] = []            # (slot, logical page, page id) not yet on the device

    @property
    def bytes_per_token(self) -> int:
        return self.num_planes * self.kv_heads * (self.head_dim + self.v_dim) * self.pages.element_size()

    def plane(self, index: int) -> Optional[torch.Tensor]:
        """[pages, 2, kv_heads, page_size, head_dim] — what the attention kernels of this library
        take; None for a group whose keys and values differ in width (use ``key_pages`` /
        ``value_pages``)."""
        return self.pages[index] if self.v_dim == self.head_dim else None

    def key_pages(self, index: int) -> torch.Tensor:
        """[pages, kv_heads, page_size, k_dim]: a view of the key rows of every page of a plane."""
        if self.v_dim == self.head_dim:
            return self.pages[index][:, 0]
        n = self.kv_heads * self.page_size * self.head_dim
        return self.pages[index][:, :n].unflatten(1, (self.kv_heads, self.page_size, self.head_dim))

    def value_pages(self, index: int) -> torch.Tensor:
        """[pages, kv_heads, page_size, v_dim]: a view of the value rows of every page of a plane."""
        if self.v_dim == self.head_dim:
            return self.pages[index][:, 1]
        n = self.kv_heads * self.page_size * self.head_dim
        return self.pages[index][:, n:].unflatten(1, (self.kv_heads, self.page_size, self.v_dim))

    # ---- planning ---------------------------------------------------------------------
    def dead_before(self, start_pos: int) -> int:
        """First logical page that a step feeding positions from ``start_pos`` on can still
        read.  Without a window every page stays.  With a window W the plane that lags most
        reads keys from (start_pos - lag) - W + 1 on."""
        if self.window is None:
            return 0
        lowest = start_pos - self.max_lag - self.window + 1
        return max(0, lowest) // self.page_size

    def pages_to_grow(self, slot: int, new_len: int) -> int:
        need_end = (new_len + self.page_size - 1) // self.page_size
        return max(0, need_end - self.end[slot])

    def pages_freed_by(self, slot: int, start_pos: int) -> int:
        return max(0, min(self.dead_before(start_pos), self.end[slot]) - self.first[slot])

    # ---- mutation ---------------------------------------------------------------------
    def trim(self, slot: int, start_pos: int) -> int:
        """Give back pages wholly behind the window of a step that starts at ``start_pos``."""
        upto = min(self.dead_before(start_pos), self.end[slot])
        n = 0
        freed: List[int] = []
        for lp in range(self.first[slot], upto):
            page = int(self.table_host[slot, lp])
            self.pool.release(page)
            self.table_host[slot, lp] = -1
            self.pending.append((slot, lp, -1))
            freed.append(page)
            n += 1
        self.first[slot] = max(self.first[slot], upto)
        self._poison(freed)
        return n

    def grow(self, slot: int, new_len: int) -> None:
        need_end = (new_len + self.page_size - 1) // self.page_size
        if need_end > self.max_pages_per_slot:
            raise CacheError(f"{new_len} tokens exceed the block table ({self.max_pages_per_slot} pages "
                             f"of {self.page_size})")
        if need_end - self.end[slot] > self.pool.free:
            raise OutOfPages(f"group {self.gid}: need {need_end - self.end[slot]} pages, {self.pool.free} free")
        first_new = self.end[slot]
        if need_end > first_new:
            # one write into the host table for all new pages (a prompt portion takes many at once)
            pages = [self.pool.allocate() for _ in range(first_new, need_end)]
            self.table_host[slot, first_new:need_end] = torch.tensor(pages, dtype=torch.int32)
            self.pending.extend((slot, first_new + i, page) for i, page in enumerate(pages))
        self.end[slot] = max(self.end[slot], need_end)

    def release_slot(self, slot: int) -> None:
        a, b = self.first[slot], self.end[slot]
        if b > a:
            freed = self.table_host[slot, a:b].tolist()
            for page in freed:
                self.pool.release(page)
            self.table_host[slot, a:b] = -1
            self.pending.extend((slot, lp, -1) for lp in range(a, b))
            self._poison(freed)
        self.first[slot] = 0
        self.end[slot] = 0

    def _poison(self, pages: List[int]) -> None:
        """Debugging mode: overwrite pages that were just given back, in every plane.  The fill is
        ordered on the stream after the steps that still read them and before any step that takes
        them again."""
        if self.poison and pages:
            idx = torch.tensor(pages, dtype=torch.int64, device=self.pages.device)
            self.pages.index_fill_(1, idx, POISON)

    def held(self, slot: int) -> int:
        return self.end[slot] - self.first[slot]

    def take_pending(self) -> List[tuple]:
        p, self.pending = self.pending, []
        return p


def group_planes(specs: Sequence[Optional[KVSpec]]):
    """Group the kv specs of the schedule entries: returns ([group key], [PlaneRef or None]).
    Entries with equal (kv_heads, key width, value width, window) share a group."""
    keys: List[tuple] = []
    lags: Dict[tuple, List[int]] = {}
    refs: List[Optional[PlaneRef]] = []
    for s in specs:
        if s is None:
            refs.append(None)
            continue
        k = s.group_key()
        if k not in lags:
            keys.append(k)
            lags[k] = []
        refs.append(PlaneRef(keys.index(k), len(lags[k])))
        lags[k].append(s.lag)
    return keys, lags, refs
