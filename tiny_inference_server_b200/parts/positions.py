"""Position encodings."""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
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

    @classmethod
    def from_config(cls, cfg):
        return cls(cfg.head_dim, cfg.rope_theta, cfg.max_context)

    def tables(self):
        i = torch.arange(0, self.rotary_dim // 2, dtype=torch.float64)
        inv = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * i / self.rotary_dim)
        ang = torch.outer(torch.arange(self.max_positions, dtype=torch.float64), inv)
        return torch.cos(ang).to(torch.float32), torch.sin(ang).to(torch.float32)

    def load(self, tensors, ctx: BuildContext) -> None:
        cos, sin = self.tables()
        self.cos = cos.to(ctx.device).contiguous()
        self.sin = sin.to(ctx.device).contiguous()

    def encode_and_store(self, qkv, step, *, num_heads, kv_heads, head_dim, plane, block_table, page_size) -> None:
        """One kernel: rotate queries (in place) and keys in float32 and write keys and values of
        every row into its page (upstream does the three in turn: main_models_new.py:75-80,
        108-112)."""
        ops.rope_kv_write(qkv, step.positions, step.row_slot, self.cos, self.sin, plane, block_table, num_heads,
                          kv_heads, head_dim, page_size, step.fault, interleaved=self.interleaved,
                          write_kv=plane is not None)


    def fused_rotary(self):
        if self.interleaved or self.rotary_dim != self.head_dim:
            return None
        return self.cos, self.sin


class RotaryInterleaved(RotaryHalf):
    """Pairs (2i, 2i+1) instead of (i, i + rot/2); the same angles."""

    def __init__(self, head_dim: int, theta: float, max_positions: int, rotary_dim: Optional[int] = None,
                 prefix: str = ""):
        super().__init__(head_dim, theta, max_positions, rotary_dim, interleaved=True, prefix=prefix)


register_part("position", "rope_half", RotaryHalf)
register_part("position", "rope_interleaved", RotaryInterleaved)
