"""Position encodings."""
from __future__ import annotations

from typing import Optional

import torch

from ..registry import register_part
from .base import BuildContext, PositionEncoding


class RotaryHalf(PositionEncoding):
    """Rotary encoding with the two halves of a head paired, (i, i + rot/2), as upstream
    (``precompute_rope_fast`` and ``rotate_half``, main_models_new.py:63-80):
    angle[pos, i] = pos * theta^(-2i/rot).  Tables of cos and sin, ``[positions, rot/2]``
    float32; the angles are formed in float64 on the host so that a table entry is the
    correctly rounded value.  ``rotary_dim`` below the head size leaves the rest of each
    head unrotated; ``interleaved`` pairs (2i, 2i+1) instead."""

    def __init__(self, head_dim: int, theta: float, max_positions: int, rotary_dim: Optional[int] = None,
                 interleaved: bool = False, prefix: str = ""):
        super().__init__(prefix)
        self.head_dim = head_dim
        self.rotary_dim = head_dim if rotary_dim is None else rotary_dim
        if self.rotary_dim % 2 or not (0 < self.rotary_dim <= head_dim):
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {head_dim}")
        self.theta = float(theta)
        self.max_positions = max_positions
        self.interleaved = interleaved
        self.cos: Optional[torch.Tensor] = None
        self.sin: Optional[torch.Tensor] = None

    def tables(self):
        i = torch.arange(0, self.rotary_dim // 2, dtype=torch.float64)
        inv = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * i / self.rotary_dim)
        ang = torch.outer(torch.arange(self.max_positions, dtype=torch.float64), inv)
        return torch.cos(ang).to(torch.float32), torch.sin(ang).to(torch.float32)

    def load(self, tensors, ctx: BuildContext) -> None:
        cos, sin = self.tables()
        self.cos = cos.to(ctx.device).contiguous()
        self.sin = sin.to(ctx.device).contiguous()


class RotaryInterleaved(RotaryHalf):
    def __init__(self, head_dim: int, theta: float, max_positions: int, rotary_dim: Optional[int] = None,
                 prefix: str = ""):
        super().__init__(head_dim, theta, max_positions, rotary_dim, interleaved=True, prefix=prefix)


register_part("position", "rope_half", RotaryHalf)
register_part("position", "rope_interleaved", RotaryInterleaved)
