"""The cache manager: request slots, their pages in every group, their fixed-size state.

Upstream keeps the per-request bookkeeping on its ``Request`` and ``User`` objects
(``server.py:76-98``, ``block_table.py:66-86``): page ids, how many positions are fed,
and for each MTP head the hidden rows not yet consumed.  Here a live request owns a
*slot*: row ``slot`` of every group's block table, and row ``slot`` of every state
tensor.  State tensors are fixed-size per request (``[slots, *shape]``); the pending
row of each MTP head lives there, and so would the state of a recurrent mixer.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from ..parts.base import KVSpec, StateSpec
from .pages import CacheError, CacheGroup, OutOfPages, PlaneRef, group_planes


class CacheManager:
    def __init__(self, kv_specs: Sequence[Optional[KVSpec]], state_specs: Dict[str, StateSpec], *,
                 page_size: int, num_pages: int, max_slots: int, max_positions: int, dtype: torch.dtype,
                 device, debug_poison: bool = False):
        self.device = torch.device(device)
        self.page_size = page_size
        self.max_slots = max_slots
        self.max_positions = max_positions
        keys, lags, self.plane_refs = group_planes(kv_specs)
        self.groups: List[CacheGroup] = [
            CacheGroup(g, k[0], k[1], k[3], lags[k], page_size, num_pages, max_slots, max_positions, dtype,
                       self.device, v_dim=k[2], poison=debug_poison)
            for g, k in enumerate(keys)
        ]
        self.states: Dict[str, torch.Tensor] = {
            name: torch.zeros((max_slots, *spec.shape), dtype=spec.dtype, device=self.device)
            for name, spec in state_specs.items()
        }
        self._free_slots = list(range(max_slots - 1, -1, -1))
        self._live = [False] * max_slots
        self.length = [0] * max_slots            # tokens fed to the slot so far

    # ---- sizes -----------------------------------------------------------------------
    @staticmethod
    def bytes_per_page(kv_specs: Sequence[Optional[KVSpec]], page_size: int, elem_size: int) -> int:
        """Bytes that one page id costs over all groups (a request holds the same number of
        pages in each group unless a window gives some back)."""
        return sum(s.kv_heads * (s.key_dim + s.value_dim) * page_size * elem_size for s in kv_specs if s is not None)

    @property
    def num_pages(self) -> int:
        return min(g.pool.num_pages for g in self.groups) if self.groups else 0

    def free_pages(self) -> int:
        """Free pages of the tightest group."""
        return min(g.pool.free for g in self.groups) if self.groups else 1 << 30

    def live_slots(self) -> List[int]:
        return [s for s in range(self.max_slots) if self._live[s]]

    # ---- slots -----------------------------------------------------------------------
    def admit(self) -> int:
        """A slot for a new request: no pages yet, state zero."""
        if not self._free_slots:
            raise CacheError("no free request slot")
        slot = self._free_slots.pop()
        self._live[slot] = True
        self.length[slot] = 0
        for t in self.states.values():
            t[slot].zero_()
        return slot

    def has_free_slot(self) -> bool:
        return bool(self._free_slots)

    def release(self, slot: int) -> None:
        """Give back everything the slot holds."""
        self._require(slot)
        for g in self.groups:
            g.release_slot(slot)
        self._live[slot] = False
        self.length[slot] = 0
        self._free_slots.append(slot)

    def _require(self, slot: int) -> None:
        if not (0 <= slot < self.max_slots) or not self._live[slot]:
            raise CacheError(f"slot {slot} is not live")

    # ---- pages -----------------------------------------------------------------------
    def pages_needed(self, slot: int, n_new: int) -> int:
        """Pages the tightest group must still have free so that ``n_new`` more tokens of
        ``slot`` fit, counting what a window would give back first."""
        self._require(slot)
        start = self.length[slot]
        need = 0
        for g in self.groups:
            grow = g.pages_to_grow(slot, start + n_new)
            if g.window is not None:
                grow -= g.pages_freed_by(slot, start)
            need = max(need, grow)
        return max(0, need)

    def pages_for_tokens(self, n_tokens: int) -> int:
        return (n_tokens + self.page_size - 1) // self.page_size

    def extend(self, slot: int, n_new: int) -> int:
        """Make room for ``n_new`` tokens after the slot's current length and advance the
        length; returns the position of the first new token.  Either every group grows or
        none does (``OutOfPages``)."""
        self._require(slot)
        start = self.length[slot]
        new_len = start + n_new
        if new_len > self.max_positions:
            raise CacheError(f"slot {slot}: {new_len} tokens exceed the context limit {self.max_positions}")
        for g in self.groups:
            grow = g.pages_to_grow(slot, new_len)
            if grow and grow - g.pages_freed_by(slot, start) > g.pool.free:
                raise OutOfPages(f"group {g.gid}: {grow} pages needed, {g.pool.free} free")
        for g in self.groups:
            if g.window is not None:
                g.trim(slot, start)
            if new_len > g.end[slot] * g.page_size:
                g.grow(slot, new_len)
        self.length[slot] = new_len
        return start

    def truncate(self, slot: int, new_len: int) -> None:
        """Forget tokens from ``new_len`` on; their cache entries are overwritten when the
        positions are fed again (upstream's position-addressed slots, block_table.py:75-80).
        Pages are kept."""
        self._require(slot)
        if not (0 <= new_len <= self.length[slot]):
            raise CacheError(f"slot {slot}: cannot truncate {self.length[slot]} tokens to {new_len}")
        for g in self.groups:
            if g.dead_before(new_len) < g.first[slot]:
                raise CacheError(f"slot {slot}: group {g.gid} has already given back pages that a step from "
                                 f"position {new_len} would read")
        self.length[slot] = new_len

    def pages_held(self, slot: int) -> int:
        return max((g.held(slot) for g in self.groups), default=0)

    # ---- device block tables ---------------------------------------------------------
    def pending_updates(self):
        """[(group, slot, logical page, page id)] not yet written to the device tables."""
        out = []
        for g in self.groups:
            out += [(g.gid, s, lp, p) for (s, lp, p) in g.take_pending()]
        return out

    def sync_tables(self) -> None:
        """Write pending block-table changes to the device (one small copy per touched slot)."""
        for g in self.groups:
            touched = sorted({s for (s, _, _) in g.take_pending()})
            for s in touched:
                g.table_dev[s].copy_(g.table_host[s], non_blocking=True)

    # ---- invariants ------------------------------------------------------------------
    def check(self) -> None:
        """No page lost, held twice or freed twice; block tables agree with the pools."""
        for g in self.groups:
            g.pool.check()
            seen = set()
            for s in range(self.max_slots):
                row = g.table_host[s].tolist()
                for lp, p in enumerate(row):
                    inside = self._live[s] and g.first[s] <= lp < g.end[s]
                    if inside:
                        if p < 0:
                            raise CacheError(f"group {g.gid} slot {s}: page {lp} missing")
                        if p in seen:
                            raise CacheError(f"group {g.gid}: page {p} held twice")
                        seen.add(p)
                    elif p != -1:
                        raise CacheError(f"group {g.gid} slot {s}: stale entry {p} at {lp}")
            if len(seen) + g.pool.free != g.pool.num_pages:
                raise CacheError(f"group {g.gid}: {len(seen)} held + {g.pool.free} free != {g.pool.num_pages}")

    def drained(self) -> bool:
        return all(g.pool.free == g.pool.num_pages for g in self.groups) and not any(self._live)
