"""Trace replay: feed given token ids through the model step by step and write logits.

Nothing is sampled.  The replay drives the engine's own model, step function, cache
manager and kernels — the ones generation uses; it has no forward pass, cache or loader
of its own.

Input, one JSON object per line::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries``: for each request its next tokens and the places among them whose logits are
wanted; all entries of a step run as one batch.  ``end``: requests that are finished
after this step; what they hold is given back.  For a step in which something is wanted
``<out>/<step>.f32`` holds the logits at the wanted places, in the order of the entries and
of ``want``, as little-endian float32 ``[wanted, vocab]``.  After every step ``done <step>``
is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Dict, IO, Iterable, Optional

import numpy as np
import torch

from .config.engine_config import EngineConfig
from .engine.batch import StepEntry
from .engine.runner import ModelRunner

#: requests live at a time that a replay is sized for unless told otherwise
MAX_LIVE = 8


class TraceReplayer:
    def __init__(self, runner: ModelRunner, out_dir: str, write_aux: bool = False):
        self.runner = runner
        self.out_dir = out_dir
        self.write_aux = write_aux
        self.slots: Dict[str, int] = {}
        os.makedirs(out_dir, exist_ok=True)

    def run_step(self, obj: dict) -> None:
        step_id = obj["step"]
        entries = []
        for e in obj.get("entries", []):
            rid = str(e["id"])
            if rid not in self.slots:
                self.slots[rid] = self.runner.add_request()
            entries.append(StepEntry(self.slots[rid], list(e["tokens"]), list(e.get("want", []))))
        if entries:
            out = self.runner.step(entries)
            if out.main.shape[0] > 0:
                self._write(os.path.join(self.out_dir, f"{step_id}.f32"), out.main)
                if self.write_aux:
                    for i, (lg, ok) in enumerate(zip(out.aux, out.aux_valid)):
                        lg = torch.where(ok[:, None], lg, torch.full_like(lg, float("nan")))
                        self._write(os.path.join(self.out_dir, f"{step_id}.mtp{i}.f32"), lg)
            self.runner.check_fault()
        for rid in obj.get("end", []):
            rid = str(rid)
            if rid in self.slots:
                self.runner.release(self.slots.pop(rid))

    @staticmethod
    def _write(path: str, logits: torch.Tensor) -> None:
        arr = logits.detach().to(torch.float32).cpu().numpy().astype("<f4", copy=False)
        tmp = path + ".tmp"
        with open(tmp, "wb") as f:
            f.write(np.ascontiguousarray(arr).tobytes())
        os.replace(tmp, path)

    def run(self, lines: Iterable[str], done: Optional[IO[str]] = None) -> None:
        for line in lines:
            line = line.strip()
            if not line:
                continue
            obj = json.loads(line)
            self.run_step(obj)
            if done is not None:
                done.write(f"done {obj['step']}\n")
                done.flush()


def pages_for(max_tokens: int, page_size: int, max_live: int) -> int:
    """Pages that hold ``max_tokens`` tokens of live requests, each request's count having been
    rounded up to a multiple of 64.  A page size that divides 64 wastes nothing.  Any other
    needs up to ceil(64 / page_size) pages for each 64 tokens of a request when it is smaller
    than 64, and one page more per live request when it is larger (the request's count is
    then rounded up to whole pages instead)."""
    if 64 % page_size == 0:
        return max(1, max_tokens // page_size + (1 if max_tokens % page_size else 0))
    if page_size < 64:
        return max(1, (max_tokens + 63) // 64 * ((64 + page_size - 1) // page_size))
    return max(1, (max_tokens + page_size - 1) // page_size + max_live)


def make_runner(model_dir: str, dtype: str, max_tokens: int, page_size: int = 16, mtp: bool = False,
                device: str = "cuda:0", cuda_graphs: bool = True, max_live: int = MAX_LIVE,
                debug_poison: bool = False) -> ModelRunner:
    """A runner whose cache pool is made for ``max_tokens`` tokens (``pages_for``), so that a
    trace which ends and starts requests uses pages again."""
    eng = EngineConfig(dtype=dtype, page_size=page_size, num_pages=pages_for(max_tokens, page_size, max_live),
                       max_batch=max_live, mtp=mtp, cuda_graphs=cuda_graphs, device=device,
                       debug_poison=debug_poison)
    return ModelRunner.from_folder(model_dir, eng)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens that live requests hold at any time; sizes the cache pool")
    ap.add_argument("--page-size", type=int, default=16, help="tokens per cache page")
    ap.add_argument("--max-live", type=int, default=MAX_LIVE, help="most requests live at a time")
    ap.add_argument("--mtp", action="store_true", help="also run the MTP heads and write <step>.mtp<i>.f32")
    args = ap.parse_args(argv)
    if args.page_size <= 0 or args.max_live <= 0:
        ap.error("--page-size and --max-live must be positive")
    print("[trace_run] loading model and kernels ...", file=sys.stderr, flush=True)
    runner = make_runner(args.model, args.dtype, args.max_tokens, args.page_size, args.mtp, max_live=args.max_live)
    from .kernels import ops
    ops.library()
    print("[trace_run] ready", file=sys.stderr, flush=True)
    TraceReplayer(runner, args.out, write_aux=args.mtp).run(sys.stdin, sys.stdout)
    return 0


if __name__ == "__main__":
    sys.exit(main())
