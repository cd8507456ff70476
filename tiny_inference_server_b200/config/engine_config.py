"""Engine options: what the upstream project keeps as module constants and Scheduler
arguments (``server.py:16-19``: ``POOL_BYTES, TOKENS_PER_BLOCK, MAX_BATCH, DEVICE``;
``server.py:106``: ``max_batch, max_context, spec, plan``)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .model_config import ConfigError


@dataclass
class EngineConfig:
    dtype: str = "bfloat16"            # "bfloat16": serving kernels; "float32": everything in true 32-bit
    page_size: int = 16                # tokens per page (upstream TOKENS_PER_BLOCK, server.py:17)
    num_pages: Optional[int] = None    # pages of every cache group; None: derived from pool_bytes
    pool_bytes: int = 4 * 1024 ** 3    # upstream POOL_BYTES, server.py:16
    max_batch: int = 8                 # live requests (upstream MAX_BATCH, server.py:18)
    max_tokens_per_step: int = 2048    # token budget of one step (decode tokens + prompt portions)
    admission: str = "final"           # "final" | "cur"  (upstream plan=, server.py:107-111)
    mtp: bool = False                  # run the MTP heads beside the trunk (upstream spec=, server.py:118)
    cuda_graphs: bool = True           # replay decode-only steps from captured graphs
    max_context: Optional[int] = None  # cap below the model's max_context
    device: str = "cuda:0"
    seed: int = 0
    debug_poison: bool = False         # fill pages with NaN patterns when they are given back (debugging aid)
    profile: bool = False              # time the phases of every step (plan, upload, launch, read-back)

    def __post_init__(self):
        errs = []
        if self.dtype in ("bf16",):
            self.dtype = "bfloat16"
        if self.dtype in ("fp32", "float"):
            self.dtype = "float32"
        if self.dtype not in ("bfloat16", "float32"):
            errs.append(f"dtype must be bfloat16 or float32, got {self.dtype!r}")
        if self.page_size <= 0:
            errs.append(f"page_size must be positive, got {self.page_size}")
        if self.num_pages is not None and self.num_pages <= 0:
            errs.append(f"num_pages must be positive, got {self.num_pages}")
        if self.max_batch <= 0:
            errs.append(f"max_batch must be positive, got {self.max_batch}")
        if self.max_tokens_per_step <= 0:
            errs.append(f"max_tokens_per_step must be positive, got {self.max_tokens_per_step}")
        if self.admission not in ("final", "cur"):
            errs.append(f"admission must be 'final' or 'cur', got {self.admission!r}")
        if errs:
            raise ConfigError("; ".join(errs))
