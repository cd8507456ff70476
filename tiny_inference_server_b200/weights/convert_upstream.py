"""Converts a checkpoint of the upstream project into a model folder of this engine.

    python -m tiny_inference_server_b200.weights.convert_upstream CKPT.pt --config CONFIG.json --out DIR

Upstream saves one pickle with two *positional* lists (``load_ckpt``, main_models_new.py:235-249):
``master_2d`` holds, in the order of ``named_parameters()``, every 2-D parameter whose name does not
contain "embed"; ``master_1d`` every 1-D parameter and the embedding matrix.  MTP heads register after
``rms_out``, so a model with fewer heads than were trained takes a prefix of both lists.  This engine
reads tensors by name from safetensors, so the converter rebuilds that order from the configuration,
gives every tensor its name, checks every shape, and writes ``config.json`` and ``model.safetensors``.
Nothing else changes: weights keep their ``(in, out)`` layout, no tensor is fused or transposed (the
engine's parts build their device layouts when they load).  ``CONFIG.json`` may use upstream's field
names (``D_MODEL, N_HEAD, NUM_GROUPS, ...``, Config/config.py:11-23).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Dict, List, Tuple

import torch

_BLOCK = ("att.q_proj.weight", "att.kv_proj.weight", "att.rms_norm_att.scale", "att.linear_proj.weight",
          "ffn.swig.linear1.weight", "ffn.swig.linear2.weight", "ffn.fc.weight", "rms_norm_ffn.scale")


def upstream_parameter_names(num_layers: int, num_mtp_heads: int) -> List[str]:
    """``named_parameters()`` of upstream's ``Transformer`` in registration order
    (main_models_new.py:83-89, 139-144, 155-161, 174-187)."""
    names = ["embedding.weight"]
    for l in range(num_layers):
        names += [f"transformer_block_list.{l}.{n}" for n in _BLOCK]
    names.append("rms_out.scale")
    for i in range(num_mtp_heads):
        pre = f"mtp_heads_list.{i}."
        names += [pre + "proj.weight", pre + "rms_embed.scale", pre + "rms_out.scale"]
        names += [pre + "trans_block." + n for n in _BLOCK]
    return names


def split_names(names: List[str], shapes: Dict[str, Tuple[int, ...]]) -> Tuple[List[str], List[str]]:
    """The names that ``master_2d`` and ``master_1d`` hold, in order (main_models_new.py:238-239)."""
    two = [n for n in names if len(shapes[n]) == 2 and "embed" not in n]
    one = [n for n in names if len(shapes[n]) == 1 or "embed" in n]
    return two, one


def convert(ckpt: dict, cfg, dtype: torch.dtype = torch.bfloat16) -> Dict[str, torch.Tensor]:
    """{tensor name: tensor} for the model of ``cfg`` (a ``GqaMtpConfig`` with tied output matrix) from
    upstream's two lists.  Raises ``WeightError`` naming what does not fit."""
    from ..registry import build_model
    from .loader import WeightError
    if not cfg.tie_word_embeddings:
        raise WeightError("upstream's model ties the output matrix to the embedding; the configuration does not")
    expected = build_model(cfg).expected_tensors()
    shapes = {n: tuple(s.shape) for n, s in expected.items()}
    names = upstream_parameter_names(cfg.num_layers, cfg.num_mtp_heads)
    if set(names) != set(shapes):
        raise WeightError(f"the configuration's model has other tensors than upstream's: "
                          f"{sorted(set(names) ^ set(shapes))[:6]} ...")
    out: Dict[str, torch.Tensor] = {}
    problems = []
    for key, which in zip(("master_2d", "master_1d"), split_names(names, shapes)):
        have = ckpt.get(key)
        if have is None:
            raise WeightError(f"the checkpoint has no list {key!r}")
        if len(have) < len(which):
            problems.append(f"{key} holds {len(have)} tensors, the model needs {len(which)}")
            continue
        for n, t in zip(which, have):            # a prefix when fewer MTP heads are wanted than were trained
            if tuple(t.shape) != shapes[n]:
                problems.append(f"{n}: checkpoint {tuple(t.shape)}, configuration {shapes[n]}")
            else:
                out[n] = t.detach().to(dtype).contiguous()
    if problems:
        raise WeightError("the checkpoint does not fit the configuration: " + "; ".join(problems[:8]) +
                          (f"; and {len(problems) - 8} more" if len(problems) > 8 else ""))
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="convert_upstream", description=__doc__.split("\n\n")[0])
    ap.add_argument("checkpoint", help="upstream's pickle with master_2d and master_1d")
    ap.add_argument("--config", required=True, help="config.json of the model that was trained")
    ap.add_argument("--out", required=True, help="model folder to write")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    args = ap.parse_args(argv)
    from safetensors.torch import save_file

    from ..config.model_config import ConfigError, write_config_json
    from ..registry import config_from_dict
    from .loader import WeightError
    try:
        with open(args.config) as f:
            cfg = config_from_dict(json.load(f))
        cfg.torch_dtype = args.dtype
        # upstream's own format: a pickle, so only load files you trust
        ckpt = torch.load(args.checkpoint, map_location="cpu", weights_only=False)
        tensors = convert(ckpt, cfg, torch.bfloat16 if args.dtype == "bfloat16" else torch.float32)
    except (ConfigError, WeightError, OSError) as e:
        print(f"convert_upstream: error: {e}", file=sys.stderr)
        return 2
    os.makedirs(args.out, exist_ok=True)
    write_config_json(args.out, cfg)
    save_file(tensors, os.path.join(args.out, "model.safetensors"))
    print(f"wrote {args.out}: {len(tensors)} tensors, step {int(ckpt.get('opt_step', 0))}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
