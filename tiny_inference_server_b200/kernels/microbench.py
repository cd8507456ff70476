"""Runs single kernels at the shapes of a model, for timing and for profiler captures.

    python -m tiny_inference_server_b200.kernels.microbench attention --batch 8 --context 4096
    python -m tiny_inference_server_b200.kernels.microbench attention-prefill --tokens 2048
    python -m tiny_inference_server_b200.kernels.microbench rowwise --tokens 2048
    python -m tiny_inference_server_b200.kernels.microbench gemm --rows 8        (weight-streaming kernel)
    python -m tiny_inference_server_b200.kernels.microbench gemm --rows 4096     (tcgen05 kernel, above 64 rows)
    python -m tiny_inference_server_b200.kernels.microbench prefill --tokens 2048 --layers 4
    python -m tiny_inference_server_b200.kernels.microbench sampling --rows 8 --vocab 49152
    python -m tiny_inference_server_b200.kernels.microbench all

``--reps N --no-timing`` launches the kernel N times and exits (a profiler attaches to that);
without it the kernels are timed with CUDA events, replayed from a CUDA graph that holds 40
launches over buffers larger than L2 (so a time includes the gap between dependent kernels,
as inside a decode step).  Default sizes are the upstream 0.9B model's: width 1536, 12 query
and 3 kv heads of 128, SwiGLU 4096.
"""
from __future__ import annotations

import argparse
import sys
import tempfile

import torch

from . import ops


def _graph_time(fn, n=40):
    fn(0)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(n):
            fn(i)
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / n * 1e3


class _Step:
    """The little of a StepContext that the attention operation reads."""

    decode_only = True

    def __init__(self, tiles, max_position):
        self._tiles = tiles
        self.max_position = max_position
        self.min_position = max_position

    def plan(self, planner):
        return self._tiles


def attention(args):
    from .attention_plan import infer_tiles
    dev = "cuda"
    H, KVH, hd, page, ctx, B = args.heads, args.kv_heads, args.head_dim, args.page_size, args.context, args.batch
    pages_per = (ctx + page - 1) // page
    num_pages = B * pages_per
    n_planes = max(2, min(12, (400 << 20) // max(1, B * ctx * 2 * KVH * hd * 2)))
    planes = [torch.randn(num_pages, 2, KVH, page, hd, device=dev, dtype=torch.bfloat16) for _ in range(n_planes)]
    table = torch.arange(num_pages, dtype=torch.int32, device=dev).reshape(B, pages_per).contiguous()
    positions = torch.full((B,), ctx - 1, dtype=torch.int32, device=dev)
    slots = torch.arange(B, dtype=torch.int32, device=dev)
    qkv = torch.randn(B, (H + 2 * KVH) * hd, device=dev, dtype=torch.bfloat16)
    out = torch.empty(B, H * hd, device=dev, dtype=torch.bfloat16)
    fault = torch.zeros(4, dtype=torch.int32, device=dev)
    step = _Step(infer_tiles(positions, slots, H // KVH), ctx - 1)
    rotary = None
    if args.rotary:          # as in a decode step: the kernel rotates q and k and writes the cache itself
        rotary = (torch.ones(ctx, hd // 2, device=dev), torch.zeros(ctx, hd // 2, device=dev))

    def run(i):
        ops.paged_attention(qkv, out, planes[i % n_planes], table, positions, slots, H, KVH, hd, page, None, fault, step,
                            rotary=rotary)

    kv_bytes = B * ctx * 2 * KVH * hd * 2
    if args.no_timing:
        for i in range(args.reps):
            run(i)
        torch.cuda.synchronize()
        print(f"attention batch {B} context {ctx}: {args.reps} launches, fault {int(fault[0])}")
        return
    t = _graph_time(run)
    print(f"attention decode  batch {B:3d} context {ctx}: {t:8.2f} us  {kv_bytes / t / 1e3:8.1f} GB/s of keys and values")


def attention_prefill(args):
    """Attention of one portion of ``--tokens`` rows at positions start..start+tokens-1 of a prompt
    (``--start 0``: a prompt over its own keys)."""
    from .attention_plan import infer_tiles
    dev = "cuda"
    H, KVH, hd, page, n = args.heads, args.kv_heads, args.head_dim, args.page_size, args.tokens
    num_pages = (args.start + n + page - 1) // page
    planes = [torch.randn(num_pages, 2, KVH, page, hd, device=dev, dtype=torch.bfloat16) for _ in range(4)]
    table = torch.arange(num_pages, dtype=torch.int32, device=dev).reshape(1, num_pages).contiguous()
    positions = torch.arange(args.start, args.start + n, dtype=torch.int32, device=dev)
    slots = torch.zeros(n, dtype=torch.int32, device=dev)
    qkv = torch.randn(n, (H + 2 * KVH) * hd, device=dev, dtype=torch.bfloat16)
    out = torch.empty(n, H * hd, device=dev, dtype=torch.bfloat16)
    fault = torch.zeros(4, dtype=torch.int32, device=dev)
    step = _Step(infer_tiles(positions, slots, H // KVH), args.start + n - 1)
    step.min_position = args.start

    def run(i):
        ops.paged_attention(qkv, out, planes[i % 4], table, positions, slots, H, KVH, hd, page, None, fault, step)

    flops = 4 * H * hd * (n * (n + 1) / 2 + n * args.start)
    if args.no_timing:
        for i in range(args.reps):
            run(i)
        torch.cuda.synchronize()
        print(f"attention prefill {n} rows: {args.reps} launches, fault {int(fault[0])}")
        return
    ops.TC_ATTENTION_MIN_TILES = 1            # time both kernels whatever the choice would be
    for tc in (True, False):
        ops.TC_ATTENTION = tc
        t = _graph_time(run, 10)
        print(f"attention prefill {n:5d} rows, {'tcgen05 ' if tc else 'mma.sync'}: {t:8.2f} us  {flops / t / 1e6:7.1f} TFLOP/s  "
              f"fault {int(fault[0])}")
    ops.TC_ATTENTION = True


def rowwise(args):
    """The memory-bound kernels between the products, at ``--tokens`` rows of the model's widths."""
    dev = "cuda"
    n, d, F, H, KVH, hd, page = args.tokens, args.width, args.ffn, args.heads, args.kv_heads, args.head_dim, args.page_size
    bufs = 6                                                   # rotate buffers so that not everything stays in L2
    res = [torch.randn(n, d, device=dev) for _ in range(bufs)]
    delta = [torch.randn(n, d, device=dev, dtype=torch.bfloat16) for _ in range(bufs)]
    normed = torch.empty(n, d, device=dev, dtype=torch.bfloat16)
    scale = torch.ones(d, device=dev)
    t = _graph_time(lambda i: ops.add_rmsnorm(res[i % bufs], delta[i % bufs], scale, 1e-6, normed), 12)
    mb = n * d * (4 + 2 + 4 + 2) / 1e6
    print(f"add_rmsnorm    {n} x {d}: {t:7.2f} us  {mb / t * 1e3:7.1f} GB/s")
    gu = [torch.randn(n, 2 * F, device=dev, dtype=torch.bfloat16) for _ in range(bufs)]
    hid = torch.empty(n, F, device=dev, dtype=torch.bfloat16)
    t = _graph_time(lambda i: ops.swiglu(gu[i % bufs], hid, 32), 12)
    mb = n * F * 6 / 1e6
    print(f"swiglu         {n} x {F}: {t:7.2f} us  {mb / t * 1e3:7.1f} GB/s")
    qkv = [torch.randn(n, (H + 2 * KVH) * hd, device=dev, dtype=torch.bfloat16) for _ in range(bufs)]
    num_pages = (n + page - 1) // page
    plane = torch.zeros(num_pages, 2, KVH, page, hd, device=dev, dtype=torch.bfloat16)
    table = torch.arange(num_pages, dtype=torch.int32, device=dev).reshape(1, num_pages).contiguous()
    positions = torch.arange(n, dtype=torch.int32, device=dev)
    slots = torch.zeros(n, dtype=torch.int32, device=dev)
    cos = torch.ones(n, hd // 2, device=dev)
    sin = torch.zeros(n, hd // 2, device=dev)
    fault = torch.zeros(4, dtype=torch.int32, device=dev)
    t = _graph_time(lambda i: ops.rope_kv_write(qkv[i % bufs], positions, slots, cos, sin, plane, table, H, KVH, hd, page,
                                                fault), 12)
    mb = n * ((H + 2 * KVH) * hd * 2 + (H + 2 * KVH) * hd * 2) / 1e6
    print(f"rope_kv_write  {n} rows: {t:7.2f} us  {mb / t * 1e3:7.1f} GB/s")


def sampling(args):
    """The sampling kernel at ``--rows`` rows of ``--vocab`` logits, for the kinds of setting a row can have."""
    dev = "cuda"
    k, v = args.rows, args.vocab
    bufs = max(2, min(16, (300 << 20) // (k * v * 4)))
    logits = [torch.randn(k, v, device=dev) * 3 for _ in range(bufs)]
    slots = torch.arange(k, dtype=torch.int32, device=dev)
    seen = torch.zeros(k, (v + 31) // 32, dtype=torch.int32, device=dev)
    seeds = torch.arange(k, dtype=torch.int64, device=dev)
    counters = torch.zeros(k, dtype=torch.int64, device=dev)
    out = torch.empty(k, dtype=torch.int32, device=dev)
    for name, temp, top_k, top_p, pen in [("greedy", 0.0, 0, 0.0, 1.0), ("temperature", 1.0, 0, 0.0, 1.0),
                                          ("top-k 50", 1.0, 50, 0.0, 1.0), ("top-p 0.9", 1.0, 0, 0.9, 1.0),
                                          ("top-k 50, top-p 0.95, penalty 1.1", 0.8, 50, 0.95, 1.1)]:
        temps = torch.full((k,), temp, device=dev)
        top_ks = torch.full((k,), top_k, dtype=torch.int32, device=dev)
        top_ps = torch.full((k,), top_p, device=dev)
        pens = torch.full((k,), pen, device=dev)
        if args.no_timing:
            if pen == 1.0:
                continue                      # a profiler looks at the setting with everything in it
            for i in range(args.reps):
                ops.sample_rows(logits[i % bufs], temps, top_ks, top_ps, pens, slots, seen, seeds, counters, out, None)
            torch.cuda.synchronize()
            print(f"sampling {k} x {v} {name}: {args.reps} launches")
            return
        t = _graph_time(lambda i: ops.sample_rows(logits[i % bufs], temps, top_ks, top_ps, pens, slots, seen, seeds,
                                                  counters, out, None), 20)
        print(f"sampling {k} x {v}  {name:36s}: {t:7.2f} us")


def gemm(args):
    dev = "cuda"
    d, F, H, KVH, hd, n = args.width, args.ffn, args.heads, args.kv_heads, args.head_dim, args.rows
    x = torch.randn(n, d, device=dev, dtype=torch.bfloat16)
    hm = torch.randn(n, F, device=dev, dtype=torch.bfloat16)
    shapes = (("qkv", d, (H + 2 * KVH) * hd, x, False), ("o", H * hd, d, x[:, : H * hd].contiguous(), False),
              ("gate_up+swiglu", d, 2 * F, x, True), ("down", F, d, hm, False))
    for name, K, N, inp, fused in shapes:
        if args.only and args.only != name:
            continue
        ws = [torch.randn(K, N, device=dev, dtype=torch.bfloat16) for _ in range(12)]

        def mine(i):
            if n > 64:
                ops.gemm_tc(inp, ws[i % 12], swiglu=fused)
            else:
                ops.gemm_skinny(inp, ws[i % 12], swiglu=fused)

        gu = torch.empty(n, N, device=dev, dtype=torch.bfloat16) if fused else None
        half = torch.empty(n, N // 2, device=dev, dtype=torch.bfloat16) if fused else None

        def lib(i):
            if fused:
                ops.swiglu(torch.mm(inp, ws[i % 12], out=gu), half, 32)
            else:
                torch.mm(inp, ws[i % 12])

        if args.no_timing:
            for i in range(args.reps):
                mine(i)
            torch.cuda.synchronize()
            print(f"gemm {name} rows {n}: {args.reps} launches")
            continue
        a, b = _graph_time(mine), _graph_time(lib)
        mb = K * N * 2 / 1e6
        extra = ""
        if n <= 64:
            # both weight-streaming kernels, whatever the dispatch would choose: the ring, the TMA boxes
            saved = (ops.STREAM_GEMM, ops.STREAM_MIN_KC, ops.STREAM_MAX_KC, ops.STREAM_MAX_CTAS, ops.STREAM_MAX_ROWS)
            times = {}
            for label, sg in (("ring", False), ("boxes", True)):
                ops.STREAM_GEMM, ops.STREAM_MIN_KC, ops.STREAM_MAX_KC, ops.STREAM_MAX_CTAS, ops.STREAM_MAX_ROWS = \
                    sg, 0, 1 << 30, 1 << 30, 64
                if not sg or ops._stream_fits(n, K, ops._ksplit(N, K)):
                    times[label] = _graph_time(mine)
            (ops.STREAM_GEMM, ops.STREAM_MIN_KC, ops.STREAM_MAX_KC, ops.STREAM_MAX_CTAS, ops.STREAM_MAX_ROWS) = saved
            times["tcgen05 swapped"] = _graph_time(lambda i: ops.gemm_swap(inp, ws[i % 12], swiglu=fused))
            extra = "   " + "  ".join(f"{k} {v:6.2f}" for k, v in times.items())
        print(f"gemm {name:15s} rows {n:4d} {mb:6.1f} MB: this kernel {a:7.2f} us ({mb / a * 1e3:7.1f} GB/s, "
              f"{2 * n * K * N / a / 1e6:6.1f} TFLOP/s)   library {b:7.2f} us{extra}")


def prefill(args):
    """One step of ``--tokens`` prompt tokens through ``--layers`` layers of the model."""
    from ..config import EngineConfig
    from ..engine import ModelRunner, StepEntry
    from ..registry import config_from_dict
    from ..weights import write_random_model
    cfg = config_from_dict(dict(architecture="gqa_mtp_transformer", vocab_size=49152, hidden_size=args.width,
                                num_layers=args.layers, num_heads=args.heads, num_kv_heads=args.kv_heads,
                                head_dim=args.head_dim, ffn_hidden=args.ffn, max_context=4096, num_mtp_heads=0))
    with tempfile.TemporaryDirectory() as tmp:
        folder = write_random_model(tmp, cfg, seed=0)
        r = ModelRunner.from_folder(folder, EngineConfig(dtype="bfloat16", page_size=args.page_size,
                                                         num_pages=(args.tokens // args.page_size + 2) * 2,
                                                         max_batch=2, max_tokens_per_step=args.tokens))
    g = torch.Generator().manual_seed(0)
    for rep in range(max(3, args.reps)):
        ids = torch.randint(0, cfg.vocab_size, (args.tokens,), generator=g).tolist()
        s = r.add_request()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        r.step([StepEntry(s, ids, [args.tokens - 1])])
        e1.record()
        torch.cuda.synchronize()
        print(f"prefill {args.tokens} tokens, {args.layers} layers: {e0.elapsed_time(e1):.3f} ms", flush=True)
        r.release(s)


def timeline(args):
    """Where the time of a decode layer goes, from inside its kernels: the five launches of a layer (qkv, attention,
    o, gate/up, down — as the engine chains them, norms folded into the products) replayed from a graph of
    ``--layers`` layers, in a build of the kernels that stamps the global timer at named places (csrc/timeline.cuh;
    compiled for this command only).  Printed for a layer in the middle: per kernel and place the first, median
    and last CTA, in ns after the last CTA of the kernel before stored its result."""
    from . import build
    from .attention_plan import infer_tiles
    if "-DTIS_TIMELINE" not in build.NVCC_FLAGS:
        build.NVCC_FLAGS.append("-DTIS_TIMELINE")            # before the libraries are first asked for
    dev = "cuda"
    d, F, H, KVH, hd, page, ctx, B, L = (args.width, args.ffn, args.heads, args.kv_heads, args.head_dim, args.page_size,
                                         args.context, args.batch, args.layers)
    lib, alib = ops.library(), ops.attention_library(hd)
    slots = lib.tis_timeline_slots()
    pages_per = (ctx + page - 1) // page
    planes = [torch.randn(B * pages_per, 2, KVH, page, hd, device=dev, dtype=torch.bfloat16) for _ in range(L)]
    table = torch.arange(B * pages_per, dtype=torch.int32, device=dev).reshape(B, pages_per).contiguous()
    positions = torch.full((B,), ctx - 1, dtype=torch.int32, device=dev)
    rows_slot = torch.arange(B, dtype=torch.int32, device=dev)
    step = _Step(infer_tiles(positions, rows_slot, H // KVH), ctx - 1)
    rotary = (torch.ones(ctx, hd // 2, device=dev), torch.zeros(ctx, hd // 2, device=dev))
    fault = torch.zeros(4, dtype=torch.int32, device=dev)

    def w(k, n):
        return [torch.randn(k, n, device=dev, dtype=torch.bfloat16) * 0.02 for _ in range(L)]
    w_qkv, w_o, w_gu, w_down = w(d, (H + 2 * KVH) * hd), w(H * hd, d), w(d, 2 * F), w(F, d)
    norm_w = torch.ones(d, device=dev)
    stream = torch.randn(B, d, device=dev)
    names = ("qkv", "attention", "o", "gate/up", "down")
    max_ctas = 1024
    stamps = torch.zeros(L * 5, max_ctas * slots, dtype=torch.int64, device=dev)
    attn_out = torch.empty(B, H * hd, device=dev, dtype=torch.bfloat16)

    def layer(l, x):
        lib.tis_timeline_next(ops._p(stamps[l * 5 + 0]))
        qkv = ops.gemm(x, w_qkv[l])
        alib.tis_timeline_next(ops._p(stamps[l * 5 + 1]))
        ops.paged_attention(qkv, attn_out, planes[l], table, positions, rows_slot, H, KVH, hd, page, None, fault, step,
                            rotary=rotary)
        lib.tis_timeline_next(ops._p(stamps[l * 5 + 2]))
        a = ops.gemm(attn_out, w_o[l], sink=ops.ResidualSink(stream, norm_w, 1e-6))
        lib.tis_timeline_next(ops._p(stamps[l * 5 + 3]))
        h = ops.gemm_swiglu(a, w_gu[l], F, 32)
        lib.tis_timeline_next(ops._p(stamps[l * 5 + 4]))
        return ops.gemm(h, w_down[l], sink=ops.ResidualSink(stream, norm_w, 1e-6))

    def run():
        x = ops.ScaledRows(torch.randn(B, d, device=dev, dtype=torch.bfloat16),
                           torch.ones(B, (d + 63) // 64, device=dev), 1e-6)
        for l in range(L):
            x = layer(l, x)
    run()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        run()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(3):
        stamps.zero_()
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
    print(f"decode layer, {B} rows, context {ctx}: {e0.elapsed_time(e1) / L * 1e3:.2f} us a layer with the stamps "
          f"(fault words {fault.tolist()})")
    t = stamps.cpu().reshape(L * 5, max_ctas, slots)
    places = {
        "gemm": ("entry", "weights ordered", "dependency wait over", "first tile ready", "loop done", "cluster barrier passed",
                 "stored"),
        "attention": ("entry", "before the dependency wait", "dependency wait over", "first tile landed", "last tile landed",
                      "loop done", "partial results pushed", "partials of the cluster arrived", "stored"),
    }
    mid = L // 2
    prev = t[mid * 5 - 1]
    prev_end = int(prev[prev[:, 0] > 0].max())
    for k in range(5):
        rec = t[mid * 5 + k]
        rec = rec[rec[:, 0] > 0]
        kind = places["attention" if k == 1 else "gemm"]
        print(f"{names[k]} ({rec.shape[0]} CTAs): ns after the last CTA of the kernel before stored (first / median / last CTA)")
        for i, place in enumerate(kind):
            v = rec[:, i]
            v = v[v > 0] - prev_end
            if v.numel():
                print(f"  {place:32s} {int(v.min()):8d} {int(v.median()):8d} {int(v.max()):8d}")
        prev_end = int(rec[:, len(kind) - 1].max())


def main(argv=None):
    ap = argparse.ArgumentParser(prog="microbench", description=__doc__.split("\n\n")[0])
    ap.add_argument("what", choices=["attention", "attention-prefill", "rowwise", "gemm", "prefill", "sampling", "timeline",
                                     "all"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--rows", type=int, default=8)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--start", type=int, default=0, help="attention-prefill: first position of the portion")
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--only", default=None, help="gemm: one of qkv, o, gate_up+swiglu, down")
    ap.add_argument("--width", type=int, default=1536)
    ap.add_argument("--heads", type=int, default=12)
    ap.add_argument("--kv-heads", type=int, default=3)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--ffn", type=int, default=4096)
    ap.add_argument("--vocab", type=int, default=49152)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--reps", type=int, default=4)
    ap.add_argument("--no-timing", action="store_true")
    ap.add_argument("--rotary", action="store_true", help="attention: rotary encoding and cache write inside the kernel")
    args = ap.parse_args(argv)
    if args.what == "timeline":
        if args.layers < 2:
            ap.error("timeline: at least two layers (the printed one has a layer before it)")
        return timeline(args) or 0
    ops.library()
    if args.what in ("attention", "all"):
        for b in ([args.batch] if args.what == "attention" else [1, 8, 64]):
            args.batch = b
            attention(args)
    if args.what in ("attention-prefill", "all"):
        attention_prefill(args)
    if args.what in ("rowwise", "all"):
        rowwise(args)
    if args.what in ("gemm", "all"):
        for n in ([args.rows] if args.what == "gemm" else [1, 8, 16]):
            args.rows = n
            gemm(args)
    if args.what in ("prefill", "all"):
        prefill(args)
    if args.what in ("sampling", "all"):
        sampling(args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
