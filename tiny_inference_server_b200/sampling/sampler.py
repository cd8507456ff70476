"""Draws the next token of each request from its row of logits on the device.

Upstream builds the probabilities of all rows with torch ops (one sort, masks, softmax:
``batch_probs``, server.py:22-50), draws with ``torch.multinomial`` and brings the tokens
back with one ``.tolist()`` (:236-240).  Here one kernel does penalty, temperature, top-k,
top-p and the draw per row; the tokens a request has seen are a bitmap row per slot that
the kernel itself extends with the token it draws.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..kernels import ops
from .params import SamplingParams


@dataclass
class SampleSpec:
    """How to draw the token after an entry's last token: the request's options, the seed of
    its random stream and how many tokens it has drawn so far (the stream's counter)."""
    params: SamplingParams
    seed: int
    counter: int


#: int32 words per row of the packed sampling parameters (see ``Sampler.pack``)
WORDS_PER_ROW = 9


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

    # ---- parameters as int32 words, for steps whose arguments live in one fixed buffer -----
    def pack(self, specs: Sequence[Optional[SampleSpec]], slots: Sequence[int], rows: int) -> List[int]:
        """``rows`` rows of sampling parameters as ``WORDS_PER_ROW * rows`` int32 words: seeds and
        counters as 64-bit little-endian pairs first (the block must start 8-byte aligned), then
        temperature, top_p, penalty (float bits), top_k, bitmap slot.  Rows beyond ``specs``
        (padding) and entries without a spec are greedy and touch no bitmap."""
        temps, tps, pens, tks, bslots, seeds, ctrs = [], [], [], [], [], [], []
        for i in range(rows):
            sp = specs[i] if i < len(specs) else None
            if sp is None:
                temps.append(0.0); tps.append(0.0); pens.append(1.0); tks.append(0); bslots.append(-1)
                seeds.append(0); ctrs.append(0)
            else:
                p = sp.params
                temps.append(p.temperature); tps.append(p.top_p); pens.append(p.rep_penalty); tks.append(p.top_k)
                bslots.append(slots[i] if p.rep_penalty != 1.0 else -1)
                seeds.append(sp.seed & 0xFFFFFFFFFFFFFFFF); ctrs.append(sp.counter)
        f = np.array([temps, tps, pens], dtype=np.float32).view(np.int32).reshape(-1).tolist()
        u = np.array([seeds, ctrs], dtype=np.uint64).view(np.int32).reshape(-1).tolist()
        return u + f + tks + bslots

    @staticmethod
    def unpack(words: torch.Tensor, rows: int):
        """Device views of a packed block (``words`` int32, 8-byte aligned): temps, top_ps,
        penalties (float32), top_ks, slots (int32), seeds, counters (int64)."""
        u = words[: 4 * rows].view(torch.int64)
        f = words[4 * rows: 7 * rows].view(torch.float32)
        i = words[7 * rows: 9 * rows]
        return f[:rows], f[rows:2 * rows], f[2 * rows:], i[:rows], i[rows:], u[:rows], u[rows:]

    def sample_packed(self, logits: torch.Tensor, words: torch.Tensor, out: Optional[torch.Tensor] = None):
        rows = logits.shape[0]
        temps, tps, pens, tks, slots, seeds, ctrs = self.unpack(words, rows)
        if out is None:
            out = torch.empty(rows, dtype=torch.int32, device=self.device)
        ops.sample_rows(logits, temps, tks, tps, pens, slots, self.seen, seeds, ctrs, out, None)
        return out

    def sample_specs(self, logits: torch.Tensor, specs: Sequence[SampleSpec], slots: Sequence[int]) -> torch.Tensor:
        """One token per row of ``logits`` for the given specs (one upload of all parameters)."""
        rows = logits.shape[0]
        words = self.pack(specs, slots, rows)
        dev = torch.tensor(words + [0], dtype=torch.int32).to(self.device, non_blocking=True)
        return self.sample_packed(logits, dev[: WORDS_PER_ROW * rows])

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
