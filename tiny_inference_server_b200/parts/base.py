"""Interfaces of the parts a model is put together from.

A part owns its weights (by tensor name below a prefix), its sizes and constants
(constructor parameters, never read from a global) and one ``forward``.  It does not
know which model it is in, which layer it is, or how the batch was cut.

What a part may ask of the engine is declared, not taken:

* a mixer that keeps keys and values declares a :class:`KVSpec`; the cache manager
  gives it a *plane* of a paged pool and the block tables of the plane's group;
* a mixer with per-request state of fixed size declares a :class:`StateSpec`; the cache
  manager gives it a tensor ``[slots, *shape]`` whose row ``slot`` belongs to one live
  request and is zero when the request is admitted.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Optional, Tuple

import torch


@dataclass(frozen=True)
class KVSpec:
    """What a mixer needs of the paged cache.  Planes with equal specs share a group:
    one pool of pages, one block table per request."""
    kv_heads: int
    head_dim: int
    window: Optional[int] = None      # None: every earlier key; W: keys p-W+1..p
    lag: int = 0                      # the plane is filled this many positions behind the trunk

    def group_key(self):
        return (self.kv_heads, self.head_dim, self.window)


@dataclass(frozen=True)
class StateSpec:
    """Per-request state of fixed size."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class WeightSpec:
    shape: Tuple[int, ...]
    init: str = "normal"              # "normal": N(0, std) ; "ones_normal": 1 + N(0, std)
    dtype: Optional[torch.dtype] = None   # None: the model's storage dtype; int32 for integer tables


@dataclass
class BuildContext:
    """Where and in which precision a model is built."""
    device: torch.device
    dtype: torch.dtype                # compute dtype: torch.bfloat16 or torch.float32

    @property
    def fp32(self) -> bool:
        return self.dtype == torch.float32


@dataclass
class LayerBinding:
    """What one entry of the layer schedule got from the cache manager."""
    kv_plane: Optional[torch.Tensor] = None   # [pages, 2, kv_heads, page_size, head_dim]
    kv_group: Optional[int] = None            # index of the plane's group (block tables, page size)
    kv_write: bool = True                     # False: the entry reads a plane that another entry fills
    state: Optional[torch.Tensor] = None      # [slots, *StateSpec.shape]


class Part:
    """Base of every part: weights by name, placed on the device in ``load``."""

    #: whether ``forward`` may be captured in a CUDA graph: it launches the same kernels with
    #: the same arguments whatever the step holds, and reads what changes (tokens, positions,
    #: slots, tiles) from the step's device arrays only
    graph_safe = True

    def __init__(self, prefix: str = ""):
        self.prefix = prefix

    # -- weights --------------------------------------------------------------------
    def weight_specs(self) -> Dict[str, WeightSpec]:
        """Local tensor name -> spec.  The full name is ``prefix + local name``."""
        return {}

    def expected_tensors(self) -> Dict[str, WeightSpec]:
        return {self.prefix + k: v for k, v in self.weight_specs().items()}

    def load(self, tensors: Dict[str, torch.Tensor], ctx: BuildContext) -> None:
        """Take this part's tensors (full names) and build the device layouts its
        kernels want.  Called once, after every name and shape has been checked."""

    def children(self):
        return ()

    def walk(self):
        yield self
        for c in self.children():
            yield from c.walk()


class Norm(Part):
    """``forward(x) -> y`` on the 32-bit residual stream; ``add_norm`` first adds a
    pending update to the stream in place, then normalises it."""

    def forward(self, residual: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def add_norm(self, residual: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    """Turns positions into what a mixer applies to queries and keys."""


class Mixer(Part):
    """Mixes information across the positions of a request.

    ``forward(x, step, binding) -> (n, width)``: ``x`` is the normalised input of the
    ``n`` rows of this step in the compute dtype; the result is the update the block
    adds to the residual stream.  ``step`` (``engine.batch.StepContext``) says which
    request and position each row is; rows of one request are contiguous and in order.
    A mixer that walks ``step.segments`` on the host is not ``graph_safe`` (the default for
    mixers); one that leaves all of that to its kernels says so.
    """

    graph_safe = False

    def kv_spec(self) -> Optional[KVSpec]:
        return None

    def state_spec(self) -> Optional[StateSpec]:
        return None

    def tile_group_sizes(self) -> Tuple[int, ...]:
        """Query heads per kv head for which the step should plan attention tiles."""
        return ()

    def forward(self, x, step, binding: LayerBinding):
        raise NotImplementedError


class FeedForward(Part):
    """``forward(x, step) -> (n, width)``, row by row: no cache, no state."""

    def forward(self, x, step):
        raise NotImplementedError
