"""Feed-forward parts."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from ..registry import register_part
from .base import BuildContext, FeedForward, WeightSpec


class SwiGLU(FeedForward):
    """``(silu(x W1) * (x W2)) W3`` (upstream ``swiglu`` and ``ffn_router``,
    main_models_new.py:44-60); weights ``(in, out)``: W1 gate and W2 up ``(width, hidden)``,
    W3 ``(hidden, width)``.  On the device gate and up are one matrix ``(width, 2*hidden)``
    whose columns alternate in blocks of 32 gates and 32 ups (when 32 divides the hidden size;
    else all gates, then all ups), so that one 64-column strip of the product holds both
    factors of 32 outputs and the gating can be the product's epilogue."""

    accepts_scaled_rows = True
    fuses_residual = True

    def __init__(self, width: int, hidden: int, prefix: str = "", names: Optional[Dict[str, str]] = None):
        super().__init__(prefix)
        self.width = width
        self.hidden = hidden
        self.names = {"gate": "swig.linear1.weight", "up": "swig.linear2.weight", "down": "fc.weight"}
        if names:
            self.names.update(names)
        self.w_gate_up = None
        self.w_down = None
        self.block = hidden

    @classmethod
    def from_config(cls, cfg, prefix: str, layer_index: int):
        return cls(cfg.hidden_size, cfg.ffn_hidden, prefix=prefix)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {
            self.names["gate"]: WeightSpec((self.width, self.hidden)),
            self.names["up"]: WeightSpec((self.width, self.hidden)),
            self.names["down"]: WeightSpec((self.hidden, self.width)),
        }

    def load(self, tensors, ctx: BuildContext) -> None:
        gate = tensors[self.prefix + self.names["gate"]]
        up = tensors[self.prefix + self.names["up"]]
        self.block = 32 if self.hidden % 32 == 0 else self.hidden
        nb = self.hidden // self.block
        both = torch.stack([gate.reshape(self.width, nb, self.block), up.reshape(self.width, nb, self.block)], dim=2)
        self.w_gate_up = both.reshape(self.width, 2 * self.hidden).to(device=ctx.device, dtype=ctx.dtype).contiguous()
        self.w_down = tensors[self.prefix + self.names["down"]].to(device=ctx.device, dtype=ctx.dtype).contiguous()

    def forward(self, x, step=None, residual=None):
        h = ops.gemm_swiglu(x, self.w_gate_up, self.hidden, self.block)
        return ops.gemm(h, self.w_down, sink=residual)


register_part("ffn", "swiglu", SwiGLU)
