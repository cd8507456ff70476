"""Norms."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from ..registry import register_part
from .base import BuildContext, Norm, WeightSpec


class RMSNormL2(Norm):
    """``y = x * sqrt(width) / (||x||_2 + eps) * scale`` in float32, eps added to the L2
    norm itself (upstream ``rms_norm``, main_models_new.py:31-42, where eps is the
    constant 2e-8; here it is a parameter)."""

    def __init__(self, width: int, eps: float, prefix: str = "", weight_name: str = "scale"):
        super().__init__(prefix)
        self.width = width
        self.eps = float(eps)
        self.weight_name = weight_name
        self.scale: Optional[torch.Tensor] = None
        self.out_dtype = torch.float32

    @classmethod
    def from_config(cls, cfg, prefix: str):
        return cls(cfg.hidden_size, cfg.rms_norm_eps, prefix=prefix)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.weight_name: WeightSpec((self.width,), init="ones_normal")}

    def load(self, tensors, ctx: BuildContext) -> None:
        self.scale = tensors[self.prefix + self.weight_name].to(device=ctx.device, dtype=torch.float32).contiguous()
        self.out_dtype = ctx.dtype

    def add_norm(self, residual: torch.Tensor, delta: Optional[torch.Tensor]) -> torch.Tensor:
        out = torch.empty(residual.shape, dtype=self.out_dtype, device=residual.device)
        return ops.add_rmsnorm(residual, delta, self.scale, self.eps, out)

    def forward(self, residual: torch.Tensor) -> torch.Tensor:
        return self.add_norm(residual, None)

    def sink(self, values: torch.Tensor):
        # the factor of a row, sqrt(width) / (||row|| + eps), is what the products apply themselves
        return ops.ResidualSink(values, self.scale, self.eps, norm=self)


register_part("norm", "rmsnorm_l2", RMSNormL2)
