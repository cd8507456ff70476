"""Random weights: a model folder (``config.json``, ``model.safetensors``) from a
configuration and a seed.

Upstream initialises by module (``linear_swig`` N(0, 1/in), ``linear_proj``
N(0, 1/(2*in*L)), embedding N(0, 1/d), norm scales 1: main_models_new.py:16-17,25-26,34,178).
For tests and benchmarks every matrix is drawn N(0, std) with one std, and norm scales
1 + N(0, std) so that a forgotten scale shows.  Values are drawn in float32 by a CPU
generator, tensor after tensor in the model's own order, and rounded once to the storage
dtype: the same configuration and seed give the same file everywhere.
"""
from __future__ import annotations

import os
from typing import Dict

import torch

from ..config.model_config import write_config_json
from ..parts.base import WeightSpec

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def random_tensors(expected: Dict[str, WeightSpec], seed: int, std: float = 0.02,
                   dtype: torch.dtype = torch.bfloat16) -> Dict[str, torch.Tensor]:
    gen = torch.Generator(device="cpu")
    gen.manual_seed(int(seed))
    out = {}
    for name, spec in expected.items():
        if spec.dtype is not None and not spec.dtype.is_floating_point:
            out[name] = torch.zeros(spec.shape, dtype=torch.int32)
            continue
        t = torch.randn(spec.shape, generator=gen, dtype=torch.float32) * std
        if spec.init == "ones_normal":
            t = t + 1.0
        elif spec.init == "ones":
            t = torch.ones(spec.shape)
        elif spec.init == "zeros":
            t = torch.zeros(spec.shape)
        out[name] = t.to(spec.dtype or dtype).contiguous()
    return out


def write_random_model(folder: str, cfg, seed: int, std: float = 0.02) -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``cfg`` under ``folder``."""
    from safetensors.torch import save_file

    from ..registry import build_model

    model = build_model(cfg)
    dtype = _DTYPES[getattr(cfg, "torch_dtype", "bfloat16")]
    tensors = random_tensors(model.expected_tensors(), seed, std, dtype)
    os.makedirs(folder, exist_ok=True)
    write_config_json(folder, cfg)
    save_file(tensors, os.path.join(folder, "model.safetensors"))
    return folder
