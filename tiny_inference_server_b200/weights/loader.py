"""Weights from safetensors, by tensor name.

Upstream loads one pickle of two flat lists by position (``load_ckpt``,
main_models_new.py:235-249): a list that is too short or in another order loads wrongly
without a word.  Here a model folder holds ``config.json`` and ``model.safetensors`` (or
several ``*.safetensors``); every tensor is found by its name, and one error lists all
that is missing, unexpected or of the wrong shape.

Tensors keep the dtype they are stored in: bfloat16 stays bfloat16, a tensor stored in
32-bit floating point stays so (float16, which float32 holds exactly, is widened),
integer tables become int32.  The parts then build the device layouts of the compute
dtype from them.
"""
from __future__ import annotations

import glob
import os
from typing import Dict

import torch

from ..parts.base import WeightSpec


class WeightError(RuntimeError):
    """The tensors of a model folder do not fit the model; the message lists every one."""


def read_safetensors(folder: str) -> Dict[str, torch.Tensor]:
    from safetensors import safe_open

    files = sorted(glob.glob(os.path.join(folder, "*.safetensors")))
    if not files:
        raise WeightError(f"no *.safetensors file in {folder!r}")
    out: Dict[str, torch.Tensor] = {}
    for path in files:
        with safe_open(path, framework="pt", device="cpu") as f:
            for name in f.keys():
                if name in out:
                    raise WeightError(f"tensor {name!r} appears in more than one file of {folder!r}")
                out[name] = f.get_tensor(name)
    return out


def _normalise_dtype(name: str, t: torch.Tensor, problems: list) -> torch.Tensor:
    if t.dtype in (torch.bfloat16, torch.float32, torch.int32):
        return t
    if t.dtype == torch.float16:
        return t.to(torch.float32)
    if t.dtype in (torch.int8, torch.int16, torch.int64, torch.uint8):
        return t.to(torch.int32)
    problems.append(f"{name}: dtype {t.dtype} is not supported (bfloat16, float32, float16, integers)")
    return t


def check_tensors(tensors: Dict[str, torch.Tensor], expected: Dict[str, WeightSpec], where: str = "") -> None:
    missing = [n for n in expected if n not in tensors]
    unexpected = [n for n in tensors if n not in expected]
    wrong = [f"{n}: stored {tuple(tensors[n].shape)}, model wants {tuple(expected[n].shape)}"
             for n in expected if n in tensors and tuple(tensors[n].shape) != tuple(expected[n].shape)]
    if missing or unexpected or wrong:
        lines = [f"weights{' in ' + where if where else ''} do not fit the model:"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shape ({len(wrong)}): " + "; ".join(wrong))
        raise WeightError("\n".join(lines))


def load_weights(folder: str, expected: Dict[str, WeightSpec]) -> Dict[str, torch.Tensor]:
    """Read, check against the model's expected tensors, normalise dtypes."""
    raw = read_safetensors(folder)
    check_tensors(raw, expected, where=folder)
    problems: list = []
    out = {n: _normalise_dtype(n, t, problems) for n, t in raw.items()}
    if problems:
        raise WeightError("weights in " + folder + ":\n  " + "\n  ".join(problems))
    return out
