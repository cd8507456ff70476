"""Trace replay on the GPU against the plain implementation: each request alone and
whole; most of it in one step and the last 32 tokens one by one; portions of changing
size down to two tokens; up to four live requests mixed, with so few pages that they are
used again — in float32 and bfloat16, for tiny configurations that differ in every size
and option.  Most replays run in this process through the engine's replayer; the
``bin/trace_run`` program itself is driven over pipes as well."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_model
import tiny_configs
import trace_tools
from tiny_inference_server_b200.trace import TraceReplayer, make_runner

pytestmark = pytest.mark.gpu

ROOT = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), os.pardir))
LENGTHS_WIDE = [70, 33, 150, 5, 200, 90]
LENGTHS = {"WIDE": LENGTHS_WIDE, "A": [1, 7, 16, 33, 50, 97, 64, 80, 120, 111, 70], "B": [2, 9, 31, 64, 100, 130, 77, 90, 128, 200],
           "C": [3, 40, 61, 90, 150, 70, 101, 64, 33, 88], "D": [5, 18, 47, 80, 33, 60, 90, 64, 71],
           "E": [300, 64, 129, 7, 200, 450, 90, 33], "F": [4, 50, 73, 120, 31, 150, 64, 97],
           "G": [2100]}
# float32: rounding of a float32 engine against a float64 oracle.
# bfloat16: weights are the same bfloat16 numbers on both sides; activations are rounded
# to bfloat16 between kernels (8 bits of mantissa) on logits of size ~0.1-1.
TOL = {"float32": 2e-4, "bfloat16": 3e-2}

_cache = {}


def _setup(name, tmp_path_factory):
    if name in _cache:
        return _cache[name]
    cfg, page, seed = tiny_configs.ALL[name]
    folder = tiny_configs.make_model_folder(cfg, seed, str(tmp_path_factory.mktemp(f"model{name}")))
    c = plain_model.read_config(folder)
    W = plain_model.read_weights(folder)
    prompts = tiny_configs.random_prompts(cfg["vocab_size"], LENGTHS[name], seed=100 + seed)
    seqs = {f"r{i}": p for i, p in enumerate(prompts)}
    plain = {rid: plain_model.plain_forward(c, W, toks) for rid, toks in seqs.items()}
    _cache[name] = (cfg, page, folder, seqs, plain)
    return _cache[name]


def _steps(mode, seqs):
    if mode == "whole":
        return trace_tools.trace_whole(seqs)
    if mode == "tail":
        return trace_tools.trace_tail(seqs, tail=32)
    if mode == "chunks":
        return trace_tools.trace_chunks(seqs)
    return trace_tools.trace_mixed(seqs, max_live=4)


def _compare(cfg, steps, out_dir, seqs, plain, tol, mtp=True):
    got = trace_tools.gather(steps, out_dir, cfg["vocab_size"])
    worst = 0.0
    for rid, toks in seqs.items():
        for p in range(len(toks)):
            err = float(np.abs(got[rid][p] - plain[rid]["main"][p].numpy()).max())
            assert err < tol, f"main logits of {rid} at position {p}: max error {err} (first wrong place)"
            worst = max(worst, err)
    if mtp:
        for i in range(cfg["num_mtp_heads"]):
            g = trace_tools.gather(steps, out_dir, cfg["vocab_size"], suffix=f"mtp{i}.f32")
            for rid, toks in seqs.items():
                for p in range(len(toks)):
                    hp = p - 1 - i
                    if hp < 0:
                        assert np.isnan(g[rid][p]).all()
                        continue
                    err = float(np.abs(g[rid][p] - plain[rid]["mtp"][i][hp].numpy()).max())
                    assert err < tol, f"mtp head {i} of {rid} at position {hp}: max error {err}"
    return worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F"])
@pytest.mark.parametrize("mode", ["whole", "tail", "chunks", "mixed"])
def test_replay_matches_plain(name, mode, dtype, tmp_path, tmp_path_factory):
    cfg, page, folder, seqs, plain = _setup(name, tmp_path_factory)
    steps = _steps(mode, seqs)
    max_tokens = trace_tools.max_live_tokens(steps, round_to=64)
    runner = make_runner(folder, dtype, max_tokens, page_size=page, mtp=True)
    if mode == "mixed":
        import random
        for g in runner.cache.groups:
            g.pool.shuffle(random.Random(5))
    out_dir = str(tmp_path / "out")
    TraceReplayer(runner, out_dir, write_aux=True).run(json.dumps(s) for s in steps)
    runner.cache.check()
    assert runner.cache.drained()
    if mode == "mixed":
        pool = runner.cache.groups[0].pool
        assert pool.allocations > pool.num_pages, "the trace does not use pages again"
    _compare(cfg, steps, out_dir, seqs, plain, TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "C", "E"])
def test_replay_with_poisoned_free_pages(name, dtype, tmp_path, tmp_path_factory):
    """The debugging mode that overwrites every page with a large pattern when it is given back (a request
    ends, a window has passed): nothing reads a page that its request no longer holds, so the logits of the
    mixed replay — pages used again, windows giving pages back — stay what they are."""
    from tiny_inference_server_b200.cache.pages import POISON
    cfg, page, folder, seqs, plain = _setup(name, tmp_path_factory)
    steps = _steps("mixed", seqs)
    runner = make_runner(folder, dtype, trace_tools.max_live_tokens(steps, round_to=64), page_size=page, mtp=True,
                         debug_poison=True)
    out_dir = str(tmp_path / "out")
    TraceReplayer(runner, out_dir, write_aux=True).run(json.dumps(s) for s in steps)
    assert runner.cache.drained()
    pool = runner.cache.groups[0].pool
    assert pool.allocations > pool.num_pages
    assert float(runner.cache.groups[0].pages.float().max()) == POISON       # the pool was poisoned
    _compare(cfg, steps, out_dir, seqs, plain, TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,page", [("A", 24), ("B", 5), ("D", 96)])
def test_replay_with_page_sizes_that_do_not_divide_64(name, page, dtype, tmp_path, tmp_path_factory):
    cfg, _, folder, seqs, plain = _setup(name, tmp_path_factory)
    steps = _steps("mixed", seqs)
    runner = make_runner(folder, dtype, trace_tools.max_live_tokens(steps, round_to=64), page_size=page, mtp=True,
                         max_live=4)
    out_dir = str(tmp_path / "out")
    TraceReplayer(runner, out_dir, write_aux=True).run(json.dumps(s) for s in steps)
    runner.cache.check()
    assert runner.cache.drained()
    _compare(cfg, steps, out_dir, seqs, plain, TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_steps_of_up_to_64_rows(dtype, tmp_path, tmp_path_factory):
    """Sixty requests live at once: decode steps of 33..60 rows (the graph bucket of 64 rows, 60 tiles in
    keys mode, library products at that many rows, sampling-free logits of every row) against the plain
    implementation, main and MTP logits at every position."""
    cfg, page, seed = tiny_configs.ALL["A"]
    folder = tiny_configs.make_model_folder(cfg, seed, str(tmp_path / "m"))
    c, W = plain_model.read_config(folder), plain_model.read_weights(folder)
    lengths = [3 + (7 * i) % 23 + 18 for i in range(60)]
    prompts = tiny_configs.random_prompts(cfg["vocab_size"], lengths, seed=77)
    seqs = {f"r{i}": p for i, p in enumerate(prompts)}
    plain = {rid: plain_model.plain_forward(c, W, toks) for rid, toks in seqs.items()}
    steps = trace_tools.trace_mixed(seqs, max_live=60, decode_from=0.3, skip_every=11)
    assert max(len(s["entries"]) for s in steps) > 48
    runner = make_runner(folder, dtype, trace_tools.max_live_tokens(steps, round_to=64), page_size=page, mtp=True,
                         max_live=64)
    out_dir = str(tmp_path / "out")
    TraceReplayer(runner, out_dir, write_aux=True).run(json.dumps(s) for s in steps)
    runner.cache.check()
    assert runner.cache.drained()
    assert any(key[0] == 64 and g.graph is not None for key, g in runner.graphs.graphs.items()), \
        "no decode step ran from the graph of 64 rows"
    _compare(cfg, steps, out_dir, seqs, plain, TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,live", [("A", 12), ("C", 24), ("E", 30), ("WIDE", 20)])
def test_decode_steps_of_9_to_32_rows(name, live, dtype, tmp_path, tmp_path_factory, monkeypatch):
    """Ten to thirty requests live at once: decode steps in the graph buckets of 16 and 32 rows.  In bfloat16 these
    are the rows for which the norms are folded into the products of this library (tiles of 16 and of 32 rows, the
    gating of 17..32 rows in the tcgen05 kernel with swapped operands) and the key splits of the lock-step attention
    kernel merge by pushing; main and MTP logits at every position against the plain implementation."""
    cfg, page, seed = tiny_configs.ALL[name]
    folder = tiny_configs.make_model_folder(cfg, seed, str(tmp_path / "m"))
    c, W = plain_model.read_config(folder), plain_model.read_weights(folder)
    lengths = [3 + (5 * i) % 17 + 14 for i in range(live)]
    prompts = tiny_configs.random_prompts(cfg["vocab_size"], lengths, seed=78)
    seqs = {f"r{i}": p for i, p in enumerate(prompts)}
    plain = {rid: plain_model.plain_forward(c, W, toks) for rid, toks in seqs.items()}
    steps = trace_tools.trace_mixed(seqs, max_live=live, decode_from=0.3, skip_every=7)
    rows = max(len(s["entries"]) for s in steps)
    assert 8 < rows <= 32
    runner = make_runner(folder, dtype, trace_tools.max_live_tokens(steps, round_to=64), page_size=page, mtp=True,
                         max_live=32)
    from tiny_inference_server_b200.kernels import ops
    sinks = []
    made = ops.ResidualSink.__init__
    monkeypatch.setattr(ops.ResidualSink, "__init__", lambda self, *a, **k: (sinks.append(a[0].shape[0]), made(self, *a, **k))[1])
    out_dir = str(tmp_path / "out")
    TraceReplayer(runner, out_dir, write_aux=True).run(json.dumps(s) for s in steps)
    runner.cache.check()
    assert runner.cache.drained()
    # bfloat16: steps of more than 8 rows had their norms folded into the products; float32: none
    assert (max(sinks, default=0) > 8) == (dtype == "bfloat16" and ops.FUSED_NORM), sinks[:8]
    bucket = 16 if rows <= 16 else 32
    assert any(key[0] == bucket and g.graph is not None for key, g in runner.graphs.graphs.items()), \
        f"no decode step ran from the graph of {bucket} rows"
    tol = TOL[dtype]
    if name == "WIDE" and dtype == "bfloat16":
        # the 0.9B widths: the bound relative to the largest logit, as in the replay at these sizes below
        tol = 1.5e-2 * float(max(plain[r]["main"].abs().max() for r in plain))
    _compare(cfg, steps, out_dir, seqs, plain, tol)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_across_the_context_bounds_of_the_graphs(dtype, tmp_path, tmp_path_factory):
    """Decode graphs are kept per bound on the context (512, 1024, 2048 keys, ...), each with its own plan
    of key splits.  One request decodes across three bounds — a new graph, another split plan, the same
    pages — and every logit equals the plain implementation's and the run without graphs."""
    from tiny_inference_server_b200.engine import StepEntry
    cfg, page, folder, seqs, plain = _setup("G", tmp_path_factory)
    toks, ref = seqs["r0"], plain["r0"]
    # portions up to just below a bound, then single tokens across it
    plan = [("portion", 500), ("decode", 530), ("portion", 1012), ("decode", 1040), ("portion", 2040),
            ("decode", 2075)]
    got = {}
    for graphs in (True, False):
        runner = make_runner(folder, dtype, 2304, page_size=page, mtp=True, cuda_graphs=graphs)
        slot = runner.add_request()
        fed, worst = 0, 0.0
        for kind, upto in plan:
            cuts = [upto - fed] if kind == "portion" else [1] * (upto - fed)
            for n in cuts:
                out = runner.step([StepEntry(slot, toks[fed:fed + n], [n - 1])])
                p = fed + n - 1
                worst = max(worst, float((out.main[0].float().cpu() - ref["main"][p].float()).abs().max()))
                assert bool(out.aux_valid[0][0])
                worst = max(worst, float((out.aux[0][0].float().cpu() - ref["mtp"][0][p - 1].float()).abs().max()))
                if kind == "decode":
                    got[(graphs, p)] = out.main[0].float().cpu().clone()
                fed += n
        runner.check_fault()
        runner.release(slot)
        assert worst < TOL[dtype], f"graphs {graphs}: worst error {worst}"
        if graphs:
            bounds = sorted({key[1] for key, g in runner.graphs.graphs.items() if g.graph is not None})
            assert len(bounds) >= 3 and bounds[:3] == [512, 1024, 2048], bounds
    for (graphs, p), v in got.items():
        if graphs:
            assert float((v - got[(False, p)]).abs().max()) < (2e-5 if dtype == "float32" else 3e-2), p


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", ["whole", "mixed"])
def test_replay_at_the_sizes_of_the_0_9b_model(mode, dtype, tmp_path, tmp_path_factory):
    """Two layers and one MTP head with the 0.9B model's layer sizes (width 1536, 12 query
    and 3 kv heads of 128, SwiGLU 4096, vocabulary 49152)."""
    cfg, page, folder, seqs, plain = _setup("WIDE", tmp_path_factory)
    steps = _steps(mode, seqs)
    max_tokens = trace_tools.max_live_tokens(steps, round_to=64)
    runner = make_runner(folder, dtype, max_tokens, page_size=page, mtp=True)
    out_dir = str(tmp_path / "out")
    TraceReplayer(runner, out_dir, write_aux=True).run(json.dumps(s) for s in steps)
    assert runner.cache.drained()
    # float32: the same absolute bound as for the tiny models.  bfloat16: logits reach ~4.7 here
    # (width 1536) and every activation is rounded to 8 bits of mantissa (0.4 % each time), so
    # the bound is relative to the largest logit: 1.5 %.
    scale = float(max(plain[r]["main"].abs().max() for r in plain))
    tol = TOL["float32"] if dtype == "float32" else 1.5e-2 * scale
    worst = _compare(cfg, steps, out_dir, seqs, plain, tol)
    print(f"worst error {worst:.3g} at logit scale {scale:.3g}")


def test_replay_with_the_tcgen05_products(tmp_path, tmp_path_factory, monkeypatch):
    """The same replay with every product of 128 rows or more on the tcgen05 kernel (by default
    only very long portions go there): whole prompts of 150 and 200 tokens in one step."""
    from tiny_inference_server_b200.kernels import ops
    monkeypatch.setattr(ops, "TC_MIN_ROWS", 128)
    monkeypatch.setattr(ops, "TC_PLAIN_MIN_ROWS", 128)
    cfg, page, folder, seqs, plain = _setup("WIDE", tmp_path_factory)
    steps = _steps("whole", seqs)
    runner = make_runner(folder, "bfloat16", trace_tools.max_live_tokens(steps, round_to=64), page_size=page, mtp=True)
    before = ops.calls["gemm_tc"]
    out_dir = str(tmp_path / "out")
    TraceReplayer(runner, out_dir, write_aux=True).run(json.dumps(s) for s in steps)
    runner.check_fault()
    scale = float(max(plain[r]["main"].abs().max() for r in plain))
    _compare(cfg, steps, out_dir, seqs, plain, 1.5e-2 * scale)
    # the two whole prompts of 150 and 200 tokens: per layer and MTP block five products each
    # (qkv, o, gate/up, down; the MTP input projection), none of which may have gone elsewhere
    assert ops.calls["gemm_tc"] - before >= 2 * (4 * 3 + 1), "the products did not go to the tcgen05 kernel"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_steps_from_cuda_graphs_equal_plain_launches(dtype, tmp_path, tmp_path_factory):
    """Steps of single tokens are replayed from captured graphs; the same trace without
    graphs gives the same logits to rounding, and both equal the plain implementation."""
    cfg, page, folder, seqs, plain = _setup("B", tmp_path_factory)
    steps = trace_tools.trace_mixed(seqs, max_live=4, decode_from=0.3, skip_every=0)
    max_tokens = trace_tools.max_live_tokens(steps, round_to=64)
    got = {}
    for graphs in (True, False):
        runner = make_runner(folder, dtype, max_tokens, page_size=page, mtp=True, cuda_graphs=graphs)
        out_dir = str(tmp_path / f"out{int(graphs)}")
        TraceReplayer(runner, out_dir, write_aux=True).run(json.dumps(s) for s in steps)
        if graphs:
            assert runner.graphs is not None and runner.graphs.replays > 10
        else:
            assert runner.graphs is None
        assert runner.cache.drained()
        _compare(cfg, steps, out_dir, seqs, plain, TOL[dtype])
        got[graphs] = trace_tools.gather(steps, out_dir, cfg["vocab_size"])
    for rid, toks in seqs.items():
        for p in range(len(toks)):
            err = float(np.abs(got[True][rid][p] - got[False][rid][p]).max())
            assert err < (2e-5 if dtype == "float32" else 3e-2), f"{rid} position {p}: {err}"


@pytest.mark.parametrize("name,dtype", [("E", "bfloat16"), ("E", "float32"), ("B", "float32")])
def test_portions_of_a_recurring_shape_from_cuda_graphs(name, dtype, tmp_path, tmp_path_factory):
    """Prompts cut into portions of one fixed size: the shape of the step comes back, so from its
    second occurrence on it is replayed from a captured graph (other positions, other pages, other
    slots); every logit equals the plain implementation, as without graphs."""
    from tiny_inference_server_b200.engine import StepEntry
    cfg, page, folder, seqs, plain = _setup(name, tmp_path_factory)
    chunk = 64
    got = {}
    for graphs in (True, False):
        runner = make_runner(folder, dtype, 4096, page_size=page, mtp=False, cuda_graphs=graphs)
        worst = 0.0
        for rid, toks in seqs.items():
            if len(toks) < 2 * chunk:
                continue
            slot = runner.add_request()
            for a in range(0, len(toks) - chunk + 1, chunk):
                out = runner.step([StepEntry(slot, toks[a:a + chunk], [0, chunk - 1])])
                for k, pos in enumerate((a, a + chunk - 1)):
                    err = float((out.main[k].float().cpu() - plain[rid]["main"][pos].float()).abs().max())
                    worst = max(worst, err)
                    got[(graphs, rid, pos)] = out.main[k].float().cpu().clone()
            runner.release(slot)
        runner.check_fault()
        assert worst < TOL[dtype], f"graphs {graphs}: worst error {worst}"
        if graphs:
            assert runner.step_graphs is not None and runner.step_graphs.replays >= 3
    for (graphs, rid, pos), v in got.items():
        if graphs:
            assert float((v - got[(False, rid, pos)]).abs().max()) < (2e-5 if dtype == "float32" else 3e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(dtype, tmp_path, tmp_path_factory):
    """bin/trace_run over pipes: one step at a time, the next only after ``done <step>``."""
    cfg, page, folder, seqs, plain = _setup("B", tmp_path_factory)
    steps = trace_tools.trace_mixed(seqs, max_live=4)
    max_tokens = trace_tools.max_live_tokens(steps, round_to=64)
    out_dir = str(tmp_path / "out")
    proc = subprocess.Popen([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                             "--out", out_dir, "--max-tokens", str(max_tokens)],
                            stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    for s in steps:
        proc.stdin.write(json.dumps(s) + "\n")
        proc.stdin.flush()
        line = proc.stdout.readline().strip()
        assert line == f"done {s['step']}", line
    proc.stdin.close()
    assert proc.wait(timeout=120) == 0
    _compare(cfg, steps, out_dir, seqs, plain, TOL[dtype], mtp=False)


def test_modes_agree_with_each_other_bitwise_close(tmp_path, tmp_path_factory):
    """In float32 the four ways of cutting give logits that agree far below the tolerance
    against the oracle: a fault of the cache or the batch would show here first."""
    cfg, page, folder, seqs, plain = _setup("A", tmp_path_factory)
    outs = {}
    for mode in ("whole", "tail", "chunks", "mixed"):
        steps = _steps(mode, seqs)
        runner = make_runner(folder, "float32", trace_tools.max_live_tokens(steps), page_size=page, mtp=False)
        out_dir = str(tmp_path / mode)
        TraceReplayer(runner, out_dir).run(json.dumps(s) for s in steps)
        outs[mode] = trace_tools.gather(steps, out_dir, cfg["vocab_size"])
    for mode in ("tail", "chunks", "mixed"):
        for rid, toks in seqs.items():
            for p in range(len(toks)):
                err = float(np.abs(outs[mode][rid][p] - outs["whole"][rid][p]).max())
                assert err < 2e-5, f"{mode} vs whole: {rid} position {p}: {err}"


def _random_configuration(seed):
    """A small configuration drawn from a seed: every size that a kernel depends on varies."""
    import random
    rng = random.Random(seed)
    hd = rng.choice([16, 32, 48, 64, 128])
    kvh = rng.choice([1, 2, 3])
    group = rng.choice([1, 2, 3, 4, 5, 8])
    width = 8 * rng.randint(5, 40)
    cfg = dict(architecture="gqa_mtp_transformer", vocab_size=rng.randint(50, 700), hidden_size=width,
               num_layers=rng.randint(1, 3), num_heads=kvh * group, num_kv_heads=kvh, head_dim=hd,
               ffn_hidden=8 * rng.randint(4, 60), rms_norm_eps=rng.choice([1e-5, 1e-6, 2e-8, 1e-3]),
               rope_theta=rng.choice([1e4, 5e5, 123.0]), max_context=512,
               tie_word_embeddings=rng.random() < 0.5, num_mtp_heads=rng.randint(0, 2))
    if rng.random() < 0.4:
        cfg["sliding_window"] = rng.randint(5, 150)
        cfg["full_attention_layers"] = [0] if rng.random() < 0.5 else []
    page = rng.choice([4, 8, 16, 32])
    lengths = [rng.randint(1, 260) for _ in range(5)] + [rng.randint(130, 300)]
    return cfg, page, lengths


@pytest.mark.parametrize("seed", [11, 12, 13, 14, 15, 16])
def test_replay_of_random_configurations(seed, tmp_path):
    """Configurations drawn at random (heads, groups, head sizes, widths and hidden sizes that are
    no powers of two, vocabulary, eps, rotary base, window, MTP heads, page size): mixed replay in
    float32 and bfloat16 against the plain implementation."""
    cfg, page, lengths = _random_configuration(seed)
    folder = tiny_configs.make_model_folder(cfg, seed, str(tmp_path / "model"))
    c, W = plain_model.read_config(folder), plain_model.read_weights(folder)
    prompts = tiny_configs.random_prompts(cfg["vocab_size"], lengths, seed=seed)
    seqs = {f"r{i}": p for i, p in enumerate(prompts)}
    plain = {rid: plain_model.plain_forward(c, W, toks) for rid, toks in seqs.items()}
    for dtype in ("float32", "bfloat16"):
        for mode in ("whole", "mixed"):
            steps = _steps(mode, seqs)
            runner = make_runner(folder, dtype, trace_tools.max_live_tokens(steps, round_to=64), page_size=page, mtp=True)
            out_dir = str(tmp_path / f"out_{dtype}_{mode}")
            TraceReplayer(runner, out_dir, write_aux=True).run(json.dumps(s) for s in steps)
            runner.check_fault()
            runner.cache.check()
            assert runner.cache.drained()
            scale = max(1.0, float(max(plain[r]["main"].abs().max() for r in plain)))
            tol = TOL["float32"] if dtype == "float32" else TOL["bfloat16"] * scale
            _compare(cfg, steps, out_dir, seqs, plain, tol)


def test_step_graphs_are_bounded_and_reused(tmp_path, tmp_path_factory):
    """A shape is captured at its second run and replayed from then on; no more than ``capacity``
    graphs are kept (the least recently used go), and a dropped shape is captured again later."""
    from tiny_inference_server_b200.engine import StepEntry
    cfg, page, folder, seqs, plain = _setup("E", tmp_path_factory)
    toks = seqs["r5"]                                      # 450 tokens
    runner = make_runner(folder, "float32", 2048, page_size=page, mtp=False)
    sg = runner.step_graphs
    assert sg is not None and sg.capacity == 6

    def run(n, tag):
        slot = runner.add_request()
        out = runner.step([StepEntry(slot, toks[:n], [n - 1])])
        err = float((out.main[0].float().cpu() - plain["r5"]["main"][n - 1].float()).abs().max())
        assert err < TOL["float32"], f"{n} tokens, {tag}: {err}"
        runner.release(slot)

    for rounds in range(3):                                # five shapes fit: eager, captured, replayed
        for n in (64, 72, 80, 96, 112):
            run(n, f"round {rounds}")
    assert len(sg.graphs) == 5 and sg.replays == 5
    for rounds in range(2):                                # eight shapes in turn: more than are kept
        for n in (64, 72, 80, 96, 112, 128, 144, 160):
            run(n, f"second part, round {rounds}")
        assert len(sg.graphs) <= sg.capacity
    run(160, "most recently used")                         # still there
    assert sg.replays >= 6
    runner.check_fault()
    assert runner.cache.drained()
