"""What the engine needs of a model, whatever its architecture.

A model is a list of *schedule entries* — (block, whose cache it reads) in running order;
the same block object may appear in several entries — plus whatever surrounds them
(embedding, final norm, heads).  The engine asks a model for

* ``walk_parts()``: its parts, to collect and load weights by tensor name;
* ``entries``: to give each entry its cache plane and state tensor;
* ``extra_states()``: further per-request state of fixed size, by name;
* ``forward(step, want_rows)``: logits at the wanted rows.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from ..parts.base import BuildContext, KVSpec, LayerBinding, Part, StateSpec
from ..parts.block import Block


@dataclass
class ScheduleEntry:
    block: Block
    source: Optional[int] = None          # index (into Model.entries) of the entry whose cache is read
    binding: LayerBinding = field(default_factory=LayerBinding)

    def kv_spec(self) -> Optional[KVSpec]:
        return None if self.source is not None else self.block.mixer.kv_spec()

    def state_spec(self) -> Optional[StateSpec]:
        return self.block.mixer.state_spec()


@dataclass
class StepOutput:
    """Logits of one step, float32.  ``main[j]`` belongs to the j-th wanted row.  ``aux[i][j]``
    are the logits of auxiliary head i (an MTP head) made in the same step at the same row,
    valid where ``aux_valid[i][j]``: head i, fed the token at position p, predicts the token
    at p+1 from position p-1-i, so its first 1+i rows of a request are not valid."""
    main: torch.Tensor
    aux: List[torch.Tensor] = field(default_factory=list)
    aux_valid: List[torch.Tensor] = field(default_factory=list)
    hidden: Optional[torch.Tensor] = None
    tokens: Optional[torch.Tensor] = None      # int32, one per entry that asked for a sample, in entry order


class Model:
    """Base of the registered architectures."""

    config = None
    vocab_size: int = 0
    max_positions: int = 0

    def __init__(self):
        self.entries: List[ScheduleEntry] = []

    # -- structure --------------------------------------------------------------------
    def top_parts(self) -> List[Part]:
        raise NotImplementedError

    def walk_parts(self):
        seen = set()
        for top in self.top_parts():
            for p in top.walk():
                if id(p) not in seen:
                    seen.add(id(p))
                    yield p

    def expected_tensors(self):
        out = {}
        for p in self.walk_parts():
            out.update(p.expected_tensors())
        return out

    def kv_specs(self) -> List[Optional[KVSpec]]:
        return [e.kv_spec() for e in self.entries]

    def lags(self) -> List[int]:
        return sorted({s.lag for s in self.kv_specs() if s is not None} | {0})

    def state_specs(self, ctx: BuildContext) -> Dict[str, StateSpec]:
        out = {}
        for i, e in enumerate(self.entries):
            s = e.state_spec()
            if s is not None:
                out[f"entry{i}"] = s
        out.update(self.extra_states(ctx))
        return out

    def extra_states(self, ctx: BuildContext) -> Dict[str, StateSpec]:
        return {}

    # -- life cycle -------------------------------------------------------------------
    def load(self, tensors: Dict[str, torch.Tensor], ctx: BuildContext) -> None:
        for p in self.walk_parts():
            p.load(tensors, ctx)

    def bind(self, cache) -> None:
        """Take cache planes and state tensors from the cache manager."""
        for i, e in enumerate(self.entries):
            src = i if e.source is None else e.source
            ref = cache.plane_refs[src]
            if ref is not None:
                grp = cache.groups[ref.group]
                e.binding.kv_plane = grp.plane(ref.index)
                e.binding.k_pages = grp.key_pages(ref.index)
                e.binding.v_pages = grp.value_pages(ref.index)
                e.binding.kv_group = ref.group
            e.binding.kv_write = e.source is None
            e.binding.state = cache.states.get(f"entry{i}")

    def forward(self, step, want_rows: torch.Tensor, aux: bool = False) -> StepOutput:
        raise NotImplementedError
