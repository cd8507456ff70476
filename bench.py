"""Decode and prefill throughput of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--sizes 3b,8b]
    python bench.py --impl reference        (the upstream project's own code, if installed)

A "step" is one decode step: every live request gets one token.  The default run has the
layer sizes of the upstream 0.9B model (30 layers, width 1536, 12 query and 3 kv heads of
128, SwiGLU 4096, vocabulary 49152, tied output matrix), random weights from a seed,
8 requests that each hold about 4096 tokens of (synthetic) cache, bfloat16.  It prints
one JSON line: decode tokens a second timed on the device with CUDA events (``value``),
the same through the Python entry point with host tokens in and out (``e2e``), a prefill
of 2048 tokens (replayed from the graph of its shape, and launched for the first time), the decode
step's HBM roofline, decode at batch 1, 16 and 64, at contexts 1024 and 8192 and with the two MTP heads
running beside the trunk, and the same points for the 3B- and 8B-sized members of the family
(``gqa_mtp_3b``, ``gqa_mtp_8b``: all their layers, context 8192, weights made on the device).
The step reads ~1.6 GB of weights and ~1.5 GB of cache, far more than the 126 MB L2, so
no L2 flush is needed between timed steps.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# the upstream 0.9B model (Config/config.py:11-23), its vocabulary rounded up to a multiple of 128
MODEL = dict(architecture="gqa_mtp_transformer", vocab_size=49152, hidden_size=1536, num_layers=30, num_heads=12,
             num_kv_heads=3, head_dim=128, ffn_hidden=4096, rms_norm_eps=2e-8, rope_theta=10000.0, max_context=4096,
             tie_word_embeddings=True, num_mtp_heads=2)
# two larger members of the same family (the layer sizes of Llama-3.2-3B and Llama-3-8B, with two MTP heads)
MODEL_3B = dict(architecture="gqa_mtp_transformer", vocab_size=128256, hidden_size=3072, num_layers=28, num_heads=24,
                num_kv_heads=8, head_dim=128, ffn_hidden=8192, rms_norm_eps=1e-5, rope_theta=500000.0,
                max_context=8192, tie_word_embeddings=True, num_mtp_heads=2)
MODEL_8B = dict(architecture="gqa_mtp_transformer", vocab_size=128256, hidden_size=4096, num_layers=32, num_heads=32,
                num_kv_heads=8, head_dim=128, ffn_hidden=14336, rms_norm_eps=1e-5, rope_theta=500000.0,
                max_context=8192, tie_word_embeddings=False, num_mtp_heads=2)
SIZES = {"0.9b": (MODEL, 4096), "3b": (MODEL_3B, 8192), "8b": (MODEL_8B, 8192)}
CONTEXT = 4096
PAGE = 16
PREFILL_TOKENS = 2048
# upstream's published iteration time at batch 8 without speculation: 31.7 ms on an RTX A6000
# (its README, "iteration time p50, batch 8") -> 8 / 0.0317 tokens a second
BASELINE_TOK_S = 8 / 0.0317


def metric_name(batch):
    """The same words from both arms (the model each arm ran is named in its ``config``)."""
    return f"decode tokens per second at batch {batch}, context {CONTEXT}, 0.9B GQA+MTP model, bf16, random weights"


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=float(p["hbm_gbs"]), bf16_tflops=float(p.get("bf16_tflops", 1590.0)), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm = [int(r[0]) for r in self.rows if r and r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": int(statistics.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def model_bytes_and_flops(cfg, n_layers, batch, ctx, elem=2, mtp_heads=0):
    """Bytes a decode step has to read (every weight it uses once, the cache of the live requests;
    upstream's formula, evals.py:143-153) and the flops of a 2048-token prefill that wants one row of
    logits (products 2*T*weights, causal attention 4*T^2*H*hd/2 per layer)."""
    d, H, KVH, hd, F, V = (cfg["hidden_size"], cfg["num_heads"], cfg["num_kv_heads"], cfg["head_dim"],
                           cfg["ffn_hidden"], cfg["vocab_size"])
    per_layer = d * (H + 2 * KVH) * hd + H * hd * d + 2 * d * F + F * d
    weights = n_layers * (per_layer + 2 * d) + d + V * d            # blocks, norms, final norm, output matrix
    weights += mtp_heads * (2 * d * d + per_layer + 4 * d)          # per head: input projection, one block, norms
    kv_per_token = (n_layers + mtp_heads) * 2 * KVH * hd
    decode_bytes = (weights + batch * ctx * kv_per_token) * elem
    t = PREFILL_TOKENS
    prefill_flops = 2 * t * n_layers * per_layer + n_layers * 4 * t * t * H * hd / 2 + 2 * d * V
    return decode_bytes, prefill_flops


def device_random_tensors(specs, seed, device, std=0.02):
    """Random weights made on the device (the random-weights mode of the package draws on the host and
    writes a folder, which for billions of parameters takes minutes): N(0, std), norm scales 1 + N(0, std)."""
    import torch
    g = torch.Generator(device=device).manual_seed(seed)
    out = {}
    for name, spec in specs.items():
        t = torch.empty(spec.shape, dtype=torch.float32, device=device).normal_(0.0, std, generator=g)
        if spec.init == "ones_normal":
            t += 1.0
        out[name] = t.to(spec.dtype or torch.bfloat16)
    return out


def fill_cache(runner, slots, length):
    """Synthetic cache: every slot holds ``length`` tokens of random keys and values."""
    import torch
    for s in slots:
        runner.cache.extend(s, length)
    runner.cache.sync_tables()
    g = torch.Generator(device=runner.device).manual_seed(1)
    for grp in runner.cache.groups:
        grp.pages.normal_(0.0, 0.5, generator=g)


def decode_run(runner, batch, start_len, steps, warmup, sampler_cls, count_ops, sampling=None):
    """Device time of ``steps`` decode steps at ``batch`` requests; returns (ms per step, launches per step).
    ``sampling``: keyword arguments of SamplingParams (default: greedy)."""
    import torch
    from tiny_inference_server_b200.engine import StepEntry
    from tiny_inference_server_b200.sampling import SampleSpec, SamplingParams

    slots = [runner.add_request() for _ in range(batch)]
    fill_cache(runner, slots, start_len)
    greedy = SamplingParams(**(sampling or {"temperature": 0.0}))
    gen = torch.Generator().manual_seed(2)
    feed = torch.randint(0, runner.vocab_size, (warmup + steps, batch), generator=gen).tolist()

    def one(i):
        # the step samples too (inside the captured graph); tokens stay on the device here
        return runner.step([StepEntry(s, [feed[i][j]], [0], SampleSpec(greedy, 0, i)) for j, s in enumerate(slots)])

    for i in range(warmup):
        one(i)
    torch.cuda.synchronize()
    l0 = count_ops()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for i in range(warmup, warmup + steps):
        one(i)
    ev1.record()
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1) / steps
    launches = (count_ops() - l0) / steps
    runner.check_fault()
    for s in slots:
        runner.release(s)
    return ms, launches


def e2e_run(engine, batch, start_len, steps, warmup):
    """The same through the Python entry point: host token ids in, host token ids out."""
    import torch
    from tiny_inference_server_b200.api import SamplingParams

    gen = torch.Generator().manual_seed(3)
    # prompts of a few tokens; the cache behind them is synthetic so that the context is ~4096
    reqs = [engine.submit(torch.randint(0, engine.runner.vocab_size, (4,), generator=gen).tolist(),
                          SamplingParams(max_new_tokens=warmup + steps + 8, temperature=0.0, ignore_eos=True))
            for _ in range(batch)]
    engine.step()                                        # prefill of the short prompts
    engine.drain()
    for r in reqs:                                       # lengthen every request's context
        extra = start_len - engine.runner.cache.length[r.slot]
        engine.runner.cache.extend(r.slot, extra)
        r.ids = [0] * extra + r.ids
        r.prompt_len += extra
        r.fed += extra
    engine.runner.cache.sync_tables()
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        engine.step()                                    # launches one step, reads the tokens of the one before
    engine.drain()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    return batch * steps / dt, dt / steps * 1e3


def prefill_run(runner, tokens, reps=3):
    """A prompt of ``tokens`` tokens in one step.  Returns (best, first): the best of ``reps`` runs once
    the step's shape has come back (from its second occurrence the engine replays it from a CUDA graph,
    as a server that cuts prompts at its token budget would see), and the time of the first run that
    is launched kernel by kernel after one warm-up run of the same shape with graphs off."""
    import torch
    from tiny_inference_server_b200.engine import StepEntry
    gen = torch.Generator().manual_seed(4)

    def once():
        ids = torch.randint(0, runner.vocab_size, (tokens,), generator=gen).tolist()
        s = runner.add_request()
        torch.cuda.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        runner.step([StepEntry(s, ids, [tokens - 1])])
        ev1.record()
        torch.cuda.synchronize()
        runner.release(s)
        return ev0.elapsed_time(ev1)

    graphs, runner.step_graphs = runner.step_graphs, None
    once()                                               # warms up (library handles, autotuned products)
    first = once()                                       # launched from Python, no graph
    runner.step_graphs = graphs
    best = min(once() for _ in range(reps + 1))          # the second run captures, later ones replay
    return best, first


def build_runner(cfg_dict, ctx, max_batch, mtp, seed=0):
    """A runner for ``cfg_dict`` with random weights made on the device and a pool for ``max_batch``
    requests of ``ctx`` tokens."""
    import torch
    from tiny_inference_server_b200.config import EngineConfig
    from tiny_inference_server_b200.engine import ModelRunner
    from tiny_inference_server_b200.registry import build_model, config_from_dict
    cfg = config_from_dict(dict(cfg_dict))
    tensors = device_random_tensors(build_model(cfg).expected_tensors(), seed, torch.device("cuda:0"))
    eng_cfg = EngineConfig(dtype="bfloat16", page_size=PAGE, num_pages=max_batch * (ctx // PAGE) + 8,
                           max_batch=max_batch, max_tokens_per_step=PREFILL_TOKENS, mtp=mtp)
    runner = ModelRunner(cfg, tensors, eng_cfg)
    del tensors
    return cfg, runner


def size_points(name, args, pk, count_ops):
    """Decode at batch 1 / 8 / 64 and a 2048-token prefill for one of the larger members of the family,
    each with its fraction of the roofline."""
    import gc
    import torch
    from tiny_inference_server_b200.sampling import Sampler
    cfg_dict, ctx = SIZES[name]
    out = {"layers": cfg_dict["num_layers"], "hidden": cfg_dict["hidden_size"], "heads": cfg_dict["num_heads"],
           "kv_heads": cfg_dict["num_kv_heads"], "ffn": cfg_dict["ffn_hidden"], "vocab": cfg_dict["vocab_size"],
           "tied": cfg_dict["tie_word_embeddings"], "seq_len": ctx, "mtp_heads_run": 0}
    runner = None
    try:
        cfg, runner = build_runner(cfg_dict, ctx, 64, mtp=False)
        steps = max(8, args.steps // 4)
        start_len = ctx - (steps + args.warmup) - 2
        for b in (1, 8, 64):
            ms, _ = decode_run(runner, b, start_len, steps, args.warmup, Sampler, count_ops)
            nbytes, flops = model_bytes_and_flops(cfg_dict, cfg_dict["num_layers"], b, ctx)
            out[f"decode_b{b}"] = round(b / (ms * 1e-3), 1)
            out[f"decode_b{b}_hbm_frac"] = round(nbytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        best, first = prefill_run(runner, PREFILL_TOKENS, reps=2)
        out["prefill"] = {"value": round(PREFILL_TOKENS / (best * 1e-3), 1), "tokens": PREFILL_TOKENS,
                          "ms": round(best, 3), "first_run_ms": round(first, 3),
                          "frac": round(flops / (best * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
    except Exception as e:                               # noqa: BLE001 - an extra point must not cost the headline
        out["error"] = f"{type(e).__name__}: {e}"[:200]
    del runner
    gc.collect()
    torch.cuda.empty_cache()
    return out


def reference_arm(args):
    """The upstream project's own code (an unmodified copy of its files under baseline/_ref: it is
    a folder of scripts, pip cannot install it) on the same metric: its Transformer with its own
    random initialisation in bfloat16, its block_table pool and Scheduler without speculation
    (server.py), 8 requests of ~4096 tokens of context; W warm-up and K timed calls of
    Scheduler.step(), timed on the device with CUDA events.  Prints `unavailable` if it cannot run."""
    ref = os.path.join(ROOT, "baseline", "_ref")

    def unavailable(why):
        print(json.dumps({"impl": "reference", "unavailable": why.replace("\n", " ")[:300]}))
        return 0

    if not os.path.isfile(os.path.join(ref, "server.py")):
        return unavailable("upstream is a folder of scripts without setup.py or pyproject.toml (pip cannot install "
                           "it) and no copy of its files is present under baseline/_ref")
    try:
        import torch
        if not torch.cuda.is_available():
            return unavailable("no CUDA device")
        sys.path.insert(0, ref)
        cwd = os.getcwd()
        os.chdir(ref)
        try:
            import server as S                     # upstream: Scheduler, Request, cfg
            from block_table import block_table
            from main_models_new import Transformer
        finally:
            os.chdir(cwd)
        cfg = S.cfg
        batch, steps, warmup = args.batch, args.steps, max(args.warmup, 3)
        dev = "cuda:0"
        torch.manual_seed(0)
        model = Transformer(cfg.VOCAB_SIZE, cfg.MAX_CONTEXT, cfg.MAX_FREQ, cfg.D_MODEL, cfg.N_HEAD, cfg.NUM_LAYERS,
                            cfg.FFN_HIDDEN_DIM, cfg.NUM_GROUPS, mtp_heads=cfg.MTP_HEADS).to(dev).to(torch.bfloat16)
        model.buffers_to_float()
        model.eval()
        planes = cfg.NUM_LAYERS + cfg.MTP_HEADS
        kvh, hd = cfg.N_HEAD // cfg.NUM_GROUPS, cfg.D_MODEL // cfg.N_HEAD
        page_bytes = 16 * 2 * 2 * kvh * planes * hd
        pool = block_table(planes, kvh, hd, (batch * (CONTEXT // 16 + 2)) * page_bytes, 16, dev)
        sched = S.Scheduler(model, pool, batch, cfg.MAX_CONTEXT, dev, spec=False)
        start_len = CONTEXT - (steps + warmup) - 2
        gen = torch.Generator().manual_seed(3)
        for _ in range(batch):
            ids = torch.randint(0, 47000, (start_len,), generator=gen).tolist()
            sched.submit(S.Request(ids, steps + warmup + 8, temperature=1.0, top_k=1))
        clocks = ClockSampler()
        sched.admit()
        sched.step()                               # prefill of the prompts and the first token
        for _ in range(warmup):
            sched.step()
        torch.cuda.synchronize()
        clocks.start()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        ev0.record()
        for _ in range(steps):
            sched.step()
        ev1.record()
        torch.cuda.synchronize()
        wall_ms = (time.perf_counter() - t0) / steps * 1e3
        ms = ev0.elapsed_time(ev1) / steps
        live = len(sched.active)
        value = live / (ms * 1e-3)
        print(json.dumps({
            "impl": "reference", "metric": metric_name(args.batch),
            "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
            "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": round(value / BASELINE_TOK_S, 2), "dtype": "bf16", "data": "synthetic",
            "config": {"model": "upstream_0.9B", "layers": cfg.NUM_LAYERS, "hidden": cfg.D_MODEL, "heads": cfg.N_HEAD,
                       "kv_heads": kvh, "head_dim": hd, "ffn": cfg.FFN_HIDDEN_DIM, "vocab": cfg.VOCAB_SIZE,
                       "mtp_heads_run": 0, "global_batch": live, "seq_len": CONTEXT, "page_size": 16,
                       "parallelism": "single_gpu", "speculation": False},
            # upstream's step takes host token ids and brings the sampled ids back (.tolist()): its
            # device-timed step is already end to end; the wall clock over the same steps is given too
            "e2e": {"value": round(live / (wall_ms * 1e-3), 1), "unit": "tokens/s", "ms_per_step": round(wall_ms, 4)},
            "clocks": clocks.stop()}))
        return 0
    except Exception as e:                         # noqa: BLE001 - any failure of upstream's code is reported, not raised
        return unavailable(f"upstream's code did not run here: {type(e).__name__}: {e}")


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=MODEL["num_layers"], help="fewer layers than the model (named in config)")
    ap.add_argument("--impl", default="engine", choices=["engine", "reference"])
    ap.add_argument("--no-points", action="store_true", help="skip batch 1 / 64, other contexts, MTP heads and prefill")
    ap.add_argument("--sizes", default="3b,8b", help="larger members of the family to measure too (3b, 8b; '' = none)")
    args = ap.parse_args(argv)
    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)

    import gc
    import torch
    from tiny_inference_server_b200.api import Engine
    from tiny_inference_server_b200.kernels import ops
    from tiny_inference_server_b200.sampling import Sampler

    cfg_dict = dict(MODEL, num_layers=args.layers)
    pk = peaks()
    max_batch = max(64, args.batch)
    cfg, runner = build_runner(cfg_dict, CONTEXT, max_batch, mtp=False)
    count_ops = lambda: ops.launches  # noqa: E731
    start_len = CONTEXT - (args.steps + args.warmup) - 2

    clocks = ClockSampler()
    clocks.start()
    ms, launches = decode_run(runner, args.batch, start_len, args.steps, args.warmup, Sampler, count_ops)
    clock_info = clocks.stop()
    value = args.batch / (ms * 1e-3)

    decode_bytes, prefill_flops = model_bytes_and_flops(cfg_dict, args.layers, args.batch, CONTEXT)
    achieved = decode_bytes / (ms * 1e-3) / 1e9
    out = {
        "metric": metric_name(args.batch),
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": round(value / BASELINE_TOK_S, 2), "dtype": "bf16", "data": "synthetic",
        "config": {"model": "gqa_mtp_0.9B", "layers": args.layers, "layers_of_model": MODEL["num_layers"],
                   "hidden": cfg.hidden_size, "heads": cfg.num_heads, "kv_heads": cfg.num_kv_heads,
                   "head_dim": cfg.head_dim, "ffn": cfg.ffn_hidden, "vocab": cfg.vocab_size,
                   "mtp_heads": cfg.num_mtp_heads, "mtp_heads_run": 0, "tied": True, "global_batch": args.batch,
                   "seq_len": CONTEXT, "page_size": PAGE, "parallelism": "single_gpu",
                   "l2": "inputs larger than L2", "peaks": pk["source"]},
        "gpu_launches": int(round(launches * args.steps)),
        "clocks": clock_info,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
    }

    # the same through the Python entry point
    engine = Engine(runner)
    e2e_tok_s, e2e_ms = e2e_run(engine, args.batch, start_len, args.steps, args.warmup)
    # one upload a step: rows, tiles and sampling parameters in one int32 buffer (plus, now and then, a
    # block-table row when a request opens a new page)
    h2d = max((g.static.used * 4 for g in runner.graphs.graphs.values()), default=0) if runner.graphs else 0
    d2h = args.batch * 4
    out["e2e"] = {"value": round(e2e_tok_s, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                  "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h}
    for r in list(engine.scheduler.active):
        engine.runner.release(r.slot)
    engine.scheduler.active = []

    if not args.no_points:
        points = {}
        half = max(8, args.steps // 2)
        for b in (1, 16, 64):
            pms, _ = decode_run(runner, b, start_len, half, args.warmup, Sampler, count_ops)
            nbytes, _ = model_bytes_and_flops(cfg_dict, args.layers, b, CONTEXT)
            points[f"decode_b{b}"] = round(b / (pms * 1e-3), 1)
            points[f"decode_b{b}_hbm_frac"] = round(nbytes / (pms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        # a shorter context on the same runner
        pms, _ = decode_run(runner, args.batch, 1024 - (half + args.warmup) - 2, half, args.warmup, Sampler, count_ops)
        nbytes, _ = model_bytes_and_flops(cfg_dict, args.layers, args.batch, 1024)
        points[f"decode_b{args.batch}_ctx1024"] = round(args.batch / (pms * 1e-3), 1)
        points[f"decode_b{args.batch}_ctx1024_hbm_frac"] = round(nbytes / (pms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        # the same step with a token drawn instead of the arg-max (the sampler runs inside the step's graph)
        drawn = {"temperature": 0.8, "top_k": 50, "top_p": 0.95, "rep_penalty": 1.1}
        pms, _ = decode_run(runner, args.batch, start_len, half, args.warmup, Sampler, count_ops, sampling=drawn)
        points[f"decode_b{args.batch}_top_k50_top_p95"] = round(args.batch / (pms * 1e-3), 1)
        out["points"] = points
        pf_ms, pf_first = prefill_run(runner, PREFILL_TOKENS)
        out["prefill"] = {"value": round(PREFILL_TOKENS / (pf_ms * 1e-3), 1), "tokens": PREFILL_TOKENS,
                          "ms": round(pf_ms, 3), "first_run_ms": round(pf_first, 3),
                          "frac": round(prefill_flops / (pf_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
        del engine, runner
        gc.collect()
        torch.cuda.empty_cache()
        # a longer context, and the MTP heads beside the trunk (runners of their own)
        try:
            _, r2 = build_runner(dict(cfg_dict, max_context=8192), 8192, args.batch, mtp=False)
            pms, _ = decode_run(r2, args.batch, 8192 - (half + args.warmup) - 2, half, args.warmup, Sampler, count_ops)
            nbytes, _ = model_bytes_and_flops(cfg_dict, args.layers, args.batch, 8192)
            points[f"decode_b{args.batch}_ctx8192"] = round(args.batch / (pms * 1e-3), 1)
            points[f"decode_b{args.batch}_ctx8192_hbm_frac"] = round(nbytes / (pms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
            del r2
            gc.collect()
            torch.cuda.empty_cache()
            _, r3 = build_runner(cfg_dict, CONTEXT, args.batch, mtp=True)
            pms, _ = decode_run(r3, args.batch, start_len, half, args.warmup, Sampler, count_ops)
            nbytes, _ = model_bytes_and_flops(cfg_dict, args.layers, args.batch, CONTEXT, mtp_heads=cfg.num_mtp_heads)
            points[f"decode_b{args.batch}_mtp{cfg.num_mtp_heads}"] = round(args.batch / (pms * 1e-3), 1)
            points[f"decode_b{args.batch}_mtp{cfg.num_mtp_heads}_hbm_frac"] = \
                round(nbytes / (pms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
            del r3
        except Exception as e:                           # noqa: BLE001 - an extra point must not cost the headline
            points["error"] = f"{type(e).__name__}: {e}"[:200]
        gc.collect()
        torch.cuda.empty_cache()
        for name in [x for x in args.sizes.split(",") if x]:
            if name in SIZES and name != "0.9b":
                out[f"gqa_mtp_{name}"] = size_points(name, args, pk, count_ops)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
