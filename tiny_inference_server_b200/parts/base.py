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
    one pool of pages, one block table per request.

    A page holds, for each kv head and each of its ``page_size`` positions, a key row of
    ``k_dim`` elements and a value row of ``v_dim`` elements (both ``head_dim`` unless given:
    a mixer with compressed keys, or keys and values of different widths, says so here)."""
    kv_heads: int
    head_dim: int
    window: Optional[int] = None      # None: every earlier key; W: keys p-W+1..p
    lag: int = 0                      # the plane is filled this many positions behind the trunk
    k_dim: Optional[int] = None       # elements of a key row (default head_dim)
    v_dim: Optional[int] = None       # elements of a value row (default head_dim)

    @property
    def key_dim(self) -> int:
        return self.head_dim if self.k_dim is None else self.k_dim

    @property
    def value_dim(self) -> int:
        return self.head_dim if self.v_dim is None else self.v_dim

    def group_key(self):
        return (self.kv_heads, self.key_dim, self.value_dim, self.window)


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
    kv_plane: Optional[torch.Tensor] = None   # [pages, 2, kv_heads, page_size, head_dim] (None when k_dim != v_dim)
    kv_group: Optional[int] = None            # index of the plane's group (block tables, page size)
    kv_write: bool = True                     # False: the entry reads a plane that another entry fills
    state: Optional[torch.Tensor] = None      # [slots, *StateSpec.shape]
    k_pages: Optional[torch.Tensor] = None    # [pages, kv_heads, page_size, k_dim]: the key rows of every page
    v_pages: Optional[torch.Tensor] = None    # [pages, kv_heads, page_size, v_dim]: the value rows of every page


class StepPlanner:
    """What a mixer's kernels want to know about a step beyond rows, positions and slots — for
    instance how the rows are cut into the tiles its kernel takes.  The engine calls ``plan`` on
    the host while it lays the step out, uploads the int32 arrays it returns in the same copy as
    the step's own arrays, and hands their device views to ``bind``; the mixer gets the result
    from ``step.plan(planner)``.  Planners with equal ``key`` are one planner: their arrays are
    made once per step whatever number of layers asks for them."""

    key = None

    def max_words(self, rows: int) -> int:
        """An upper bound on the total length of the arrays for a step of ``rows`` rows (sizes
        the fixed metadata buffer of a captured step)."""
        raise NotImplementedError

    def plan(self, segments):
        """``segments``: [(first row, rows)] of the step, one per request (padding rows as
        segments of one row).  Returns ({array name: list of ints}, host-side facts)."""
        raise NotImplementedError

    def plan_decode(self, rows: int):
        """``plan`` for a step of ``rows`` single-token segments (override when that is cheaper)."""
        return self.plan([(r, 1) for r in range(rows)])

    def bind(self, arrays: Dict[str, torch.Tensor], facts):
        """What the mixer wants to get: by default the device arrays and the facts as they are."""
        return arrays, facts

    def infer(self, positions: torch.Tensor, row_slot: torch.Tensor):
        """The plan from the device arrays alone (synchronises; for calls outside a step, as in
        kernel tests): consecutive rows with one slot and consecutive positions form a segment."""
        pos, slot = positions.tolist(), row_slot.tolist()
        segs = []
        for r in range(len(pos)):
            if segs and slot[r] >= 0 and slot[r] == slot[r - 1] and pos[r] == pos[r - 1] + 1:
                segs[-1] = (segs[-1][0], segs[-1][1] + 1)
            else:
                segs.append((r, 1))
        arrays, facts = self.plan(segs)
        dev = positions.device
        return self.bind({k: torch.tensor(v, dtype=torch.int32, device=dev) for k, v in arrays.items()}, facts)


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
    pending update to the stream in place, then normalises it.

    ``sink(values)``: a norm whose factor per row is a function of the row's sum of squares may return
    a ``kernels.ops.ResidualSink`` for the stream ``values``: the part before the norm then adds its
    update to the stream inside its last product and the part after applies the factor after its first
    product, so that the norm needs no kernel.  None (the default): the norm runs as a kernel of its own."""

    @classmethod
    def from_config(cls, cfg, prefix: str):
        raise NotImplementedError

    def sink(self, values: torch.Tensor):
        return None

    def forward(self, residual: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def add_norm(self, residual: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    """Turns positions into what is applied to queries and keys before they meet.

    ``encode_and_store(qkv, step, ...)``: ``qkv`` holds, per row, the queries of ``num_heads``
    heads, then the keys and then the values of ``kv_heads`` heads (``head_dim`` each).  The
    encoding is applied to queries (in place) and keys at the rows' positions
    (``step.positions``), and — when ``plane`` is given — the encoded keys and the values of every
    row are written into the row's page of the cache, in the cache's row format.  Keys are
    stored *after* encoding, so an encoding must depend on the absolute position only.
    One fused kernel does all of it for the rotary family; an encoding of another kind brings
    its own way and still ends with the cache write."""

    @classmethod
    def from_config(cls, cfg):
        raise NotImplementedError

    def encode_and_store(self, qkv: torch.Tensor, step, *, num_heads: int, kv_heads: int, head_dim: int,
                         plane: Optional[torch.Tensor], block_table: Optional[torch.Tensor], page_size: int) -> None:
        raise NotImplementedError

    def fused_rotary(self):
        """(cos, sin) tables ``[positions, head_dim / 2]`` float32 if this encoding is a rotation of
        the whole head with pairs (i, i + head_dim/2) — what the decode attention kernel can apply
        itself, together with the cache write, in place of ``encode_and_store`` — else None."""
        return None


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
    #: ``x`` may come as ``kernels.ops.ScaledRows`` (a norm's output that still lacks the factor of each row)
    accepts_scaled_rows = False
    #: ``forward`` takes ``residual=`` (a ``kernels.ops.ResidualSink`` or None); given one, it may add its update
    #: to the stream itself and return the ``ScaledRows`` its last product made instead of the update
    fuses_residual = False

    def kv_spec(self) -> Optional[KVSpec]:
        return None

    def state_spec(self) -> Optional[StateSpec]:
        return None

    @classmethod
    def from_config(cls, cfg, prefix: str, layer_index: int, lag: int, position=None):
        """Build the mixer of layer ``layer_index`` from the model configuration.  ``lag``: the
        layer belongs to a stage that runs this many positions behind the trunk; ``position``:
        the model's position encoding (a mixer that needs none ignores it)."""
        raise NotImplementedError

    def step_planners(self) -> Tuple[StepPlanner, ...]:
        """Planners whose arrays the engine should make and upload with every step."""
        return ()

    def forward(self, x, step, binding: LayerBinding):
        raise NotImplementedError


class FeedForward(Part):
    """``forward(x, step) -> (n, width)``, row by row: no cache, no state.
    ``accepts_scaled_rows`` and ``fuses_residual``: as for a mixer."""

    accepts_scaled_rows = False
    fuses_residual = False

    @classmethod
    def from_config(cls, cfg, prefix: str, layer_index: int):
        raise NotImplementedError

    def forward(self, x, step):
        raise NotImplementedError
