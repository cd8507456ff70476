"""Sampling options of a request, with upstream's names, meanings and defaults
(``Request(prompt_ids, max_new_tokens, temperature=1.0, top_k=0, top_p=0,
rep_penalty=1.0)``, server.py:79; 0 switches top-k / top-p off, 1.0 the penalty)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass
class SamplingParams:
    max_new_tokens: int = 200
    temperature: float = 1.0       # 0: greedy (upstream has no greedy switch; its tests use top_k=1)
    top_k: int = 0
    top_p: float = 0.0
    rep_penalty: float = 1.0
    seed: Optional[int] = None     # None: engine seed + request id
    ignore_eos: bool = False       # keep generating past the end-of-sequence token (benchmarks)

    def __post_init__(self):
        if self.max_new_tokens <= 0:
            raise ValueError(f"max_new_tokens must be positive, got {self.max_new_tokens}")
        if self.temperature < 0:
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")
        if self.top_k < 0:
            raise ValueError(f"top_k must be >= 0, got {self.top_k}")
        if not (0.0 <= self.top_p <= 1.0):
            raise ValueError(f"top_p must be in [0, 1], got {self.top_p}")
        if self.rep_penalty <= 0:
            raise ValueError(f"rep_penalty must be positive, got {self.rep_penalty}")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0 or self.top_k == 1
