"""Draws the next token of each request from its row of logits on the device.

Upstream builds the probabilities of all rows with torch ops (one sort, masks, softmax:
``batch_probs``, server.py:22-50), draws with ``torch.multinomial`` and brings the tokens
back with one ``.tolist()`` (:236-240).  Here one kernel does penalty, temperature, top-k,
top-p and the draw per row; the tokens a request has seen are a bitmap row per slot that
the kernel itself extends with the token it draws.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..kernels import ops
from .params import SamplingParams


class Sampler:
    def __init__(self, vocab_size: int, max_slots: int, device, seed: int = 0):
        self.vocab_size = vocab_size
        self.device = torch.device(device)
        self.seed = int(seed)
        self.words = (vocab_size + 31) // 32
        self.seen = torch.zeros((max_slots, self.words), dtype=torch.int32, device=self.device)

    def start_request(self, slot: int, params: SamplingParams, context: Sequence[int]) -> None:
        """Reset the slot's seen-token bitmap to ``context`` (prompt, or prompt and what was
        generated before a preemption).  Only requests with a penalty keep a bitmap."""
        if params.rep_penalty == 1.0:
            return
        self.seen[slot].zero_()
        if len(context):
            toks = torch.tensor(list(context), dtype=torch.int32).to(self.device)
            ops.bitmap_set(self.seen[slot], toks)

    def request_seed(self, params: SamplingParams, request_id: int) -> int:
        base = params.seed if params.seed is not None else self.seed * 1000003 + request_id
        return base & 0xFFFFFFFFFFFFFFFF

    def sample(self, logits: torch.Tensor, params: List[SamplingParams], slots: List[int], seeds: List[int],
               counters: List[int], probs_out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One token per row of ``logits`` (k, vocab) float32; returns int32 (k,) on the device."""
        k = logits.shape[0]
        f = torch.tensor([[p.temperature for p in params], [p.top_p for p in params],
                          [p.rep_penalty for p in params]], dtype=torch.float32).to(self.device, non_blocking=True)
        i = torch.tensor([[p.top_k for p in params],
                          [s if p.rep_penalty != 1.0 else -1 for p, s in zip(params, slots)]],
                         dtype=torch.int32).to(self.device, non_blocking=True)
        # seeds and counters as int64 bit patterns of the unsigned values
        u = torch.tensor([[s - (1 << 64) if s >= (1 << 63) else s for s in seeds], list(counters)],
                         dtype=torch.int64).to(self.device, non_blocking=True)
        out = torch.empty(k, dtype=torch.int32, device=self.device)
        ops.sample_rows(logits, f[0], i[0], f[1], f[2], i[1], self.seen, u[0], u[1], out, probs_out)
        return out
