"""The residual stream of a step: a float32 tensor (rows, width) and at most one update
that has not been added yet.  The pending update is added by the norm that reads the
stream next (one fused kernel), which is where every pre-norm block wants it.

A part whose last product can add to the stream itself is given a *sink* instead (``sink``); what it
hands back is the next norm's output short of one factor per row (``kernels.ops.ScaledRows``), kept
here until that norm asks for it."""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops


class ResidualStream:
    def __init__(self, values: torch.Tensor):
        assert values.dtype == torch.float32
        self.values = values
        self.pending: Optional[torch.Tensor] = None
        self.ready: Optional[ops.ScaledRows] = None

    def sink(self, norm, dtype: torch.dtype):
        """A sink for the part that runs before ``norm``, or None when this step's rows or the norm do
        not allow one.  ``dtype``: the compute dtype of the products."""
        if self.pending is not None or not ops.sink_usable(self.values, dtype):
            return None
        return norm.sink(self.values)

    def add(self, update) -> None:
        """``update``: a part's result, or the ``ScaledRows`` of a part that has added its result itself."""
        if isinstance(update, ops.ScaledRows):
            self.ready = update
            return
        self.ready = None
        if self.pending is not None:
            ops.residual_add(self.values, self.pending)
        self.pending = update

    def normed(self, norm, scaled: bool = False):
        """norm(values + pending); the sum stays in ``values``.  ``scaled``: the reader takes ``ScaledRows``."""
        ready, self.ready = self.ready, None
        if ready is not None:
            if ready.norm is norm:
                return ready if scaled else ready.dense()
            return norm.add_norm(self.values, None)        # made for another norm: the stream itself is whole
        delta, self.pending = self.pending, None
        return norm.add_norm(self.values, delta)

    def flush(self) -> torch.Tensor:
        self.ready = None
        if self.pending is not None:
            ops.residual_add(self.values, self.pending)
            self.pending = None
        return self.values
