"""The residual stream of a step: a float32 tensor (rows, width) and at most one update
that has not been added yet.  The pending update is added by the norm that reads the
stream next (one fused kernel), which is where every pre-norm block wants it."""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops


class ResidualStream:
    def __init__(self, values: torch.Tensor):
        assert values.dtype == torch.float32
        self.values = values
        self.pending: Optional[torch.Tensor] = None

    def add(self, delta: torch.Tensor) -> None:
        if self.pending is not None:
            ops.residual_add(self.values, self.pending)
        self.pending = delta

    def normed(self, norm) -> torch.Tensor:
        """norm(values + pending); the sum stays in ``values``."""
        delta, self.pending = self.pending, None
        return norm.add_norm(self.values, delta)

    def flush(self) -> torch.Tensor:
        if self.pending is not None:
            ops.residual_add(self.values, self.pending)
            self.pending = None
        return self.values
