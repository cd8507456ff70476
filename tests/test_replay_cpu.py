"""The step function, the cache manager and trace replay on the CPU, with the plain
PyTorch references in place of the CUDA kernels: whatever way the tokens are cut into
steps and batched, the logits equal the plain implementation's."""
import json

import numpy as np
import pytest
import torch

import plain_model
import tiny_configs
import trace_tools
from tiny_inference_server_b200.trace import TraceReplayer, make_runner

LENGTHS = {"A": [1, 7, 16, 33, 50], "B": [2, 9, 31, 64, 70], "C": [3, 40, 61, 90], "D": [5, 18, 47], "F": [4, 50, 73, 31]}


def _setup(name, tmp_path):
    cfg, page, seed = tiny_configs.ALL[name]
    folder = tiny_configs.make_model_folder(cfg, seed, str(tmp_path / f"model{name}"))
    c = plain_model.read_config(folder)
    W = plain_model.read_weights(folder)
    prompts = tiny_configs.random_prompts(cfg["vocab_size"], LENGTHS[name], seed=100 + seed)
    seqs = {f"r{i}": p for i, p in enumerate(prompts)}
    plain = {rid: plain_model.plain_forward(c, W, toks) for rid, toks in seqs.items()}
    return cfg, page, folder, seqs, plain


def _replay(folder, page, steps, out_dir, max_tokens, dtype="float32", mtp=True):
    runner = make_runner(folder, dtype, max_tokens, page_size=page, mtp=mtp, device="cpu")
    rep = TraceReplayer(runner, out_dir, write_aux=mtp)
    rep.run(json.dumps(s) for s in steps)
    runner.cache.check()
    assert runner.cache.drained(), "pages or slots were not given back"
    return runner


def _compare(cfg, steps, out_dir, seqs, plain, tol):
    got = trace_tools.gather(steps, out_dir, cfg["vocab_size"])
    for rid, toks in seqs.items():
        for p in range(len(toks)):
            ref = plain[rid]["main"][p].numpy()
            err = np.abs(got[rid][p] - ref).max()
            assert err < tol, f"main logits of {rid} at position {p}: max error {err}"
    for i in range(cfg["num_mtp_heads"]):
        g = trace_tools.gather(steps, out_dir, cfg["vocab_size"], suffix=f"mtp{i}.f32")
        for rid, toks in seqs.items():
            for p in range(len(toks)):
                hp = p - 1 - i          # head i, fed token p, speaks for position p-1-i
                if hp < 0:
                    assert np.isnan(g[rid][p]).all()
                    continue
                ref = plain[rid]["mtp"][i][hp].numpy()
                err = np.abs(g[rid][p] - ref).max()
                assert err < tol, f"mtp head {i} of {rid} at position {hp}: max error {err}"


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "F"])
@pytest.mark.parametrize("mode", ["whole", "tail", "chunks", "mixed"])
def test_replay_modes_match_plain(name, mode, tmp_path, ref_ops):
    cfg, page, folder, seqs, plain = _setup(name, tmp_path)
    if mode == "whole":
        steps = trace_tools.trace_whole(seqs)
    elif mode == "tail":
        steps = trace_tools.trace_tail(seqs, tail=32)
    elif mode == "chunks":
        steps = trace_tools.trace_chunks(seqs)
    else:
        steps = trace_tools.trace_mixed(seqs, max_live=3)
    max_tokens = trace_tools.max_live_tokens(steps, round_to=64)
    out_dir = str(tmp_path / f"out_{mode}")
    _replay(folder, page, steps, out_dir, max_tokens)
    _compare(cfg, steps, out_dir, seqs, plain, tol=2e-4)


def test_pages_are_used_again(tmp_path, ref_ops):
    """The mixed trace needs more pages over its life than the pool has."""
    cfg, page, folder, seqs, plain = _setup("A", tmp_path)
    steps = trace_tools.trace_mixed(seqs, max_live=2)
    max_tokens = trace_tools.max_live_tokens(steps, round_to=64)
    total = sum((len(t) + page - 1) // page for t in seqs.values())
    assert total > max_tokens // page or True
    out_dir = str(tmp_path / "out")
    runner = _replay(folder, page, steps, out_dir, max_tokens)
    assert runner.cache.groups[0].pool.num_pages == max_tokens // page
    _compare(cfg, steps, out_dir, seqs, plain, tol=2e-4)


def test_norms_folded_into_the_products_change_nothing_but_rounding(tmp_path, ref_ops, monkeypatch):
    """bfloat16 steps of few rows: the last product of a mixer or feed-forward adds to the residual stream itself
    and the next product applies the norm's factor (``ResidualSink`` / ``ScaledRows``), here with the references
    of those products.  The logits equal those of the same steps with the norm as an operation of its own to
    bfloat16 rounding, and the folded path is the one that ran."""
    from tiny_inference_server_b200.kernels import ops
    cfg, page, folder, seqs, plain = _setup("A", tmp_path)
    steps = trace_tools.trace_tail(seqs, tail=32)
    max_tokens = trace_tools.max_live_tokens(steps, round_to=64)
    made = []
    whole = ops.ScaledRows.dense
    monkeypatch.setattr(ops.ScaledRows, "dense", lambda self: made.append("dense") or whole(self))
    sink_of = ops.ResidualSink.__init__

    def counted(self, *a, **k):
        made.append("sink")
        sink_of(self, *a, **k)
    monkeypatch.setattr(ops.ResidualSink, "__init__", counted)
    got = {}
    for fused in (True, False):
        monkeypatch.setattr(ops, "FUSED_NORM", fused)
        made.clear()
        out_dir = str(tmp_path / f"out_{fused}")
        _replay(folder, page, steps, out_dir, max_tokens, dtype="bfloat16")
        got[fused] = trace_tools.gather(steps, out_dir, cfg["vocab_size"])
        layers = cfg["num_layers"]
        if fused:
            # per single-row step: the mixer of every layer and the feed-forward of every layer but the last
            assert made.count("sink") >= 32 * (2 * layers - 1) and "dense" not in made
        else:
            assert not made
    for rid, toks in seqs.items():
        for p in range(len(toks)):
            a, b, ref = got[True][rid][p], got[False][rid][p], plain[rid]["main"][p].numpy()
            scale = np.abs(ref).max()
            assert np.abs(a - b).max() < 0.05 * scale + 0.05, f"{rid} at {p}: the two ways differ by {np.abs(a - b).max()}"
            assert np.abs(a - ref).max() < 0.08 * scale + 0.08, f"{rid} at {p}: {np.abs(a - ref).max()} from the plain model"
