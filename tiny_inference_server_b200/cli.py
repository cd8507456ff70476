"""Command line: generate from token ids with a model folder or a random model.

Upstream has no options — ``python server.py`` runs ten built-in prompts with constants
edited in the file (server.py:12-19, 482-530).  The options here carry upstream's names
where it has them: ``--max-new-tokens --temperature --top-k --top-p --rep-penalty`` are the
fields of its ``Request`` (server.py:79), ``--max-batch``, ``--pool-bytes`` and
``--tokens-per-block`` its ``MAX_BATCH``, ``POOL_BYTES`` and ``TOKENS_PER_BLOCK``
(server.py:16-18), ``--plan`` its admission plan (server.py:106).

    python -m tiny_inference_server_b200.cli --model DIR --prompt-ids 5,17,3 --prompt-ids 9,9
    python -m tiny_inference_server_b200.cli --random CONFIG.json --seed 0 --write-model DIR
"""
from __future__ import annotations

import argparse
import json
import sys
import tempfile
import time


def _ids(text: str):
    return [int(t) for t in text.replace(",", " ").split()]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="tiny_inference_server_b200", description=__doc__.split("\n\n")[0])
    src = ap.add_mutually_exclusive_group(required=True)
    src.add_argument("--model", help="folder with config.json and model.safetensors")
    src.add_argument("--random", metavar="CONFIG.json", help="make random weights for this configuration")
    ap.add_argument("--seed", type=int, default=0, help="seed of random weights and of sampling")
    ap.add_argument("--write-model", metavar="DIR", help="with --random: write the model folder here and exit")
    ap.add_argument("--prompt-ids", action="append", default=[], metavar="IDS",
                    help="token ids of one prompt, separated by commas or spaces; repeatable")
    ap.add_argument("--prompt-file", help="file with one prompt per line (token ids)")
    ap.add_argument("--max-new-tokens", type=int, default=200)
    ap.add_argument("--temperature", type=float, default=1.0, help="0 = greedy")
    ap.add_argument("--top-k", type=int, default=0, help="0 = off")
    ap.add_argument("--top-p", type=float, default=0.0, help="0 = off")
    ap.add_argument("--rep-penalty", type=float, default=1.0, help="1 = off")
    ap.add_argument("--greedy", action="store_true", help="same as --temperature 0")
    ap.add_argument("--ignore-eos", action="store_true")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32", "bf16", "fp32"])
    ap.add_argument("--tokens-per-block", "--page-size", dest="page_size", type=int, default=16)
    ap.add_argument("--pool-bytes", type=int, default=4 * 1024 ** 3)
    ap.add_argument("--num-pages", type=int, default=None, help="overrides --pool-bytes")
    ap.add_argument("--max-batch", type=int, default=8)
    ap.add_argument("--max-tokens-per-step", type=int, default=2048)
    ap.add_argument("--plan", default="final", choices=["final", "cur"], help="admission plan")
    ap.add_argument("--mtp", action="store_true", help="run the MTP heads beside the trunk")
    ap.add_argument("--no-cuda-graphs", action="store_true")
    ap.add_argument("--json", action="store_true", help="print one JSON object instead of text")
    args = ap.parse_args(argv)

    from .config import ConfigError, EngineConfig
    from .kernels.build import BuildError
    from .kernels.ops import KernelError
    from .weights import WeightError
    try:
        return _run(ap, args)
    except (ConfigError, WeightError, KernelError, BuildError) as e:
        # what a user can put right (a bad config.json, tensors that do not fit it, no B200, no
        # compiler) is one line, not a traceback
        print(f"{ap.prog}: error: {e}", file=sys.stderr)
        return 2


def _run(ap, args) -> int:
    from .config import EngineConfig
    from .registry import config_from_dict
    from .weights import write_random_model

    folder = args.model
    tmp = None
    if args.random:
        with open(args.random) as f:
            cfg = config_from_dict(json.load(f))
        if args.write_model:
            write_random_model(args.write_model, cfg, args.seed)
            print(f"wrote {args.write_model}")
            return 0
    prompts = [_ids(p) for p in args.prompt_ids]
    if args.prompt_file:
        with open(args.prompt_file) as f:
            prompts += [_ids(line) for line in f if line.strip()]
    if not prompts:
        ap.error("no prompt: give --prompt-ids or --prompt-file")

    from .kernels import ops
    ops.library()                   # no CUDA device, no sm_100 GPU or no compiler: KernelError / BuildError here
    if args.random:
        tmp = tempfile.TemporaryDirectory()
        folder = write_random_model(tmp.name, cfg, args.seed)

    from .api import Engine, SamplingParams

    eng_cfg = EngineConfig(dtype=args.dtype, page_size=args.page_size, num_pages=args.num_pages,
                           pool_bytes=args.pool_bytes, max_batch=args.max_batch,
                           max_tokens_per_step=args.max_tokens_per_step, admission=args.plan, mtp=args.mtp,
                           cuda_graphs=not args.no_cuda_graphs, seed=args.seed)
    engine = Engine.from_folder(folder, eng_cfg)
    params = SamplingParams(max_new_tokens=args.max_new_tokens,
                            temperature=0.0 if args.greedy else args.temperature, top_k=args.top_k,
                            top_p=args.top_p, rep_penalty=args.rep_penalty, ignore_eos=args.ignore_eos)
    import torch

    torch.cuda.synchronize()
    t0 = time.time()
    outs = engine.generate(prompts, params)
    torch.cuda.synchronize()
    dt = time.time() - t0
    total = sum(len(o) for o in outs)
    if args.json:
        print(json.dumps({"outputs": outs, "new_tokens": total, "seconds": dt, "tokens_per_second": total / dt,
                          "stats": engine.stats()}))
    else:
        for p, o in zip(prompts, outs):
            print("PROMPT:", " ".join(map(str, p)))
            print("OUTPUT:", " ".join(map(str, o)))
        print(f"\n{total} tokens in {dt:.2f}s ({total / dt:.1f} tok/s)")
    if tmp is not None:
        tmp.cleanup()
    return 0


if __name__ == "__main__":
    sys.exit(main())
