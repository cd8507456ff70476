"""Grouped-query attention over the paged cache."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import attention_plan, ops
from ..registry import register_part
from .base import BuildContext, KVSpec, LayerBinding, Mixer, WeightSpec


class GqaAttention(Mixer):
    """q/kv projections, rotary encoding, cache write, causal attention over the cache,
    output projection (upstream ``paged_gqa``, main_models_new.py:83-136; the norm before
    and the residual add after belong to the block).

    Weights as stored upstream, ``(in, out)``: ``q_proj (width, H*hd)``,
    ``kv_proj (width, 2*KVH*hd)`` with the keys in the first half of the columns
    (main_models_new.py:104-106), ``linear_proj (H*hd, width)``.  On the device q and kv
    are one matrix so that a step makes one product for both.

    ``window``: the row at position p sees keys p-window+1..p instead of 0..p.
    ``lag``: the layer belongs to a stage that runs this many positions behind the trunk.
    """

    graph_safe = True
    accepts_scaled_rows = True
    fuses_residual = True

    def __init__(self, width: int, num_heads: int, kv_heads: int, head_dim: int, position,
                 window: Optional[int] = None, lag: int = 0, prefix: str = "",
                 names: Optional[Dict[str, str]] = None):
        super().__init__(prefix)
        if num_heads % kv_heads:
            raise ValueError(f"{num_heads} query heads are not a multiple of {kv_heads} kv heads")
        if head_dim % 16 or not (16 <= head_dim <= 256):
            raise ValueError(f"head size {head_dim}: the attention kernels take multiples of 16 from 16 to 256")
        self.width = width
        self.num_heads = num_heads
        self.kv_heads = kv_heads
        self.head_dim = head_dim
        self.window = window
        self.lag = lag
        self.position = position
        self.names = {"q": "q_proj.weight", "kv": "kv_proj.weight", "o": "linear_proj.weight"}
        if names:
            self.names.update(names)
        self.w_qkv = None
        self.w_q = None
        self.w_o = None

    @classmethod
    def from_config(cls, cfg, prefix: str, layer_index: int, lag: int, position=None):
        return cls(cfg.hidden_size, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, position,
                   window=cfg.window_of(layer_index), lag=lag, prefix=prefix)

    def children(self):
        return (self.position,)

    def kv_spec(self) -> KVSpec:
        return KVSpec(self.kv_heads, self.head_dim, self.window, self.lag)

    def step_planners(self):
        # the tiles the bfloat16 attention kernels take, for this layer's group size
        return (attention_plan.planner(self.num_heads // self.kv_heads),)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        hq, hkv = self.num_heads * self.head_dim, self.kv_heads * self.head_dim
        return {
            self.names["q"]: WeightSpec((self.width, hq)),
            self.names["kv"]: WeightSpec((self.width, 2 * hkv)),
            self.names["o"]: WeightSpec((hq, self.width)),
        }

    def load(self, tensors, ctx: BuildContext) -> None:
        q = tensors[self.prefix + self.names["q"]]
        kv = tensors[self.prefix + self.names["kv"]]
        self.w_qkv = torch.cat([q, kv], dim=1).to(device=ctx.device, dtype=ctx.dtype).contiguous()
        self.w_q = self.w_qkv[:, : self.num_heads * self.head_dim]
        self.w_o = tensors[self.prefix + self.names["o"]].to(device=ctx.device, dtype=ctx.dtype).contiguous()

    def forward(self, x, step, binding: LayerBinding, residual=None):
        n = x.shape[0]
        hq = self.num_heads * self.head_dim
        g = binding.kv_group
        table = step.block_tables[g]
        page_size = step.page_sizes[g]
        qkv = ops.gemm(x, self.w_qkv if binding.kv_write else self.w_q)
        out = torch.empty((n, hq), dtype=qkv.dtype, device=qkv.device)
        # a decode step: the attention kernel applies a rotary encoding and writes the cache itself
        rotary = self.position.fused_rotary()
        if rotary is not None and ops.rotary_fusable(qkv, step, self.num_heads, self.kv_heads, self.head_dim):
            ops.paged_attention(qkv, out, binding.kv_plane, table, step.positions, step.row_slot, self.num_heads,
                                self.kv_heads, self.head_dim, page_size, self.window, step.fault, step,
                                rotary=rotary, write_kv=binding.kv_write)
            return ops.gemm(out, self.w_o, sink=residual)
        self.position.encode_and_store(qkv, step, num_heads=self.num_heads, kv_heads=self.kv_heads,
                                       head_dim=self.head_dim, plane=binding.kv_plane if binding.kv_write else None,
                                       block_table=table, page_size=page_size)
        ops.paged_attention(qkv, out, binding.kv_plane, table, step.positions, step.row_slot, self.num_heads,
                            self.kv_heads, self.head_dim, page_size, self.window, step.fault, step)
        return ops.gemm(out, self.w_o, sink=residual)


register_part("mixer", "gqa", GqaAttention)
