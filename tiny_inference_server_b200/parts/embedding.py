"""Token embedding and the output projection onto the vocabulary."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from .base import BuildContext, Part, WeightSpec


class Embedding(Part):
    """``x = E[token]`` with no scaling (main_models_new.py:177-178,199).  The gathered rows
    start the float32 residual stream."""

    def __init__(self, vocab: int, width: int, prefix: str = "", weight_name: str = "embedding.weight"):
        super().__init__(prefix)
        self.vocab = vocab
        self.width = width
        self.weight_name = weight_name
        self.table: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.weight_name: WeightSpec((self.vocab, self.width))}

    def load(self, tensors, ctx: BuildContext) -> None:
        self.table = tensors[self.prefix + self.weight_name].to(device=ctx.device, dtype=ctx.dtype).contiguous()

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        out = torch.empty((tokens.shape[0], self.width), dtype=torch.float32, device=tokens.device)
        return ops.embed_rows(self.table, tokens, out)


class LMHead(Part):
    """``logits = h @ E^T`` with the embedding matrix (tied, main_models_new.py:225-226) or
    with a matrix of its own, ``lm_head.weight (vocab, width)``.  Logits are float32."""

    def __init__(self, vocab: int, width: int, embedding: Optional[Embedding], prefix: str = "",
                 weight_name: str = "lm_head.weight"):
        super().__init__(prefix)
        self.vocab = vocab
        self.width = width
        self.embedding = embedding            # given: tied
        self.weight_name = weight_name
        self.weight_t: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        if self.embedding is not None:
            return {}
        return {self.weight_name: WeightSpec((self.vocab, self.width))}

    def load(self, tensors, ctx: BuildContext) -> None:
        if self.embedding is None:
            w = tensors[self.prefix + self.weight_name].to(device=ctx.device, dtype=ctx.dtype).contiguous()
            self.weight_t = w.t()

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        wt = self.weight_t if self.embedding is None else self.embedding.table.t()
        return ops.gemm_f32_out(h, wt)
