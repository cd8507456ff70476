"""The plain implementation itself: against the committed outputs of the upstream
project's own model code (tests/golden/), and a few properties of its parts."""
import math
import os

import numpy as np
import pytest
import torch

import plain_model
import tiny_configs

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_tiny.npz")


def _golden_model(tmp_path):
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(os.path.dirname(GOLDEN), "make_golden.py"))
    mg = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mg)
    folder = tiny_configs.make_model_folder(mg.CFG, mg.SEED, str(tmp_path / "golden_model"))
    return mg, folder


def test_plain_equals_upstream_model_code(tmp_path):
    mg, folder = _golden_model(tmp_path)
    g = np.load(GOLDEN)
    assert g["tokens"].tolist() == mg.TOKENS and int(g["seed"][0]) == mg.SEED
    c = plain_model.read_config(folder)
    W = plain_model.read_weights(folder, torch.float64)
    out = plain_model.plain_forward(c, W, mg.TOKENS)
    # upstream ran in float32: agreement to float32 rounding
    np.testing.assert_allclose(out["main"].numpy(), g["main"], rtol=0, atol=5e-6)
    np.testing.assert_allclose(out["mtp"][0].numpy(), g["mtp0"], rtol=0, atol=5e-6)
    np.testing.assert_allclose(out["mtp"][1].numpy(), g["mtp1"], rtol=0, atol=5e-6)
    dec = plain_model.plain_forward(c, W, mg.TOKENS + [mg.NEXT], mtp=False)["main"][-1:]
    np.testing.assert_allclose(dec.numpy(), g["decode"], rtol=0, atol=5e-6)


def test_plain_attention_equals_upstream_dense_oracle(tmp_path):
    """``dense_main`` is the output of upstream's own dense oracle (test_server.py:23-45:
    ``scaled_dot_product_attention(is_causal=True)`` after ``repeat_interleave``), with none of
    this repository's attention code on its path: it pins the scale 1/sqrt(head size), the causal
    rule and query head h -> kv head h // group.  Each of the three, got wrong, must fail."""
    mg, folder = _golden_model(tmp_path)
    g = np.load(GOLDEN)
    c = plain_model.read_config(folder)
    W = plain_model.read_weights(folder, torch.float64)
    out = plain_model.plain_forward(c, W, mg.TOKENS, mtp=False)["main"].numpy()
    np.testing.assert_allclose(out, g["dense_main"], rtol=0, atol=5e-6)

    real = plain_model.plain_causal_attention

    def differs(wrong):
        plain_model.plain_causal_attention = wrong
        try:
            bad = plain_model.plain_forward(c, W, mg.TOKENS, mtp=False)["main"].numpy()
        finally:
            plain_model.plain_causal_attention = real
        return float(np.abs(bad - g["dense_main"]).max())

    H, KVH = c["num_heads"], c["num_kv_heads"]
    # query head h -> kv head h % KVH instead of h // group
    perm = [(h % KVH) * (H // KVH) + h // KVH for h in range(H)]
    inv = [perm.index(h) for h in range(H)]
    assert differs(lambda q, k, v, **kw: real(q[:, perm], k, v, **kw)[:, inv]) > 1e-4
    # another scale
    assert differs(lambda q, k, v, **kw: real(q * 1.5, k, v, **kw)) > 1e-4
    # a row that also sees the key after it
    def sees_next(q, k, v, **kw):
        o = real(q, k, v, **kw)
        o2 = real(q[:-1], k[1:], v[1:], **kw)       # row p over keys 1..p+1
        return torch.cat([0.5 * (o[:-1] + o2), o[-1:]])
    assert differs(sees_next) > 1e-4


def test_rms_norm_form():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    y = plain_model.plain_rms_norm(x, torch.ones(2, dtype=torch.float64), 1.0)
    # ||x|| = 5: x * sqrt(2) / (5 + 1)
    assert torch.allclose(y, x * math.sqrt(2) / 6)


def test_rope_is_a_rotation_and_relative():
    hd = 16
    g = torch.Generator().manual_seed(0)
    q = torch.randn(1, 1, hd, generator=g, dtype=torch.float64)
    k = torch.randn(1, 1, hd, generator=g, dtype=torch.float64)

    def rot(x, p):
        c, s = plain_model.plain_rope_angles(torch.tensor([p]), 10000.0, hd)
        return plain_model.plain_apply_rope(x, c, s)

    assert torch.allclose(rot(q, 5).norm(), q.norm())
    a = (rot(q, 9) * rot(k, 4)).sum()
    b = (rot(q, 105) * rot(k, 100)).sum()
    assert torch.allclose(a, b)


def test_causal_attention_sees_no_future_and_honours_window():
    g = torch.Generator().manual_seed(1)
    T, H, KVH, hd = 12, 4, 2, 8
    q = torch.randn(T, H, hd, generator=g, dtype=torch.float64)
    k = torch.randn(T, KVH, hd, generator=g, dtype=torch.float64)
    v = torch.randn(T, KVH, hd, generator=g, dtype=torch.float64)
    o1 = plain_model.plain_causal_attention(q, k, v)
    k2, v2 = k.clone(), v.clone()
    k2[7:] += 3
    v2[7:] -= 2
    o2 = plain_model.plain_causal_attention(q, k2, v2)
    assert torch.allclose(o1[:7], o2[:7]) and not torch.allclose(o1[7:], o2[7:])
    ow = plain_model.plain_causal_attention(q, k, v, window=3)
    k3 = k.clone()
    k3[:5] += 5                      # keys 0..4 are outside the window of positions >= 7
    ow3 = plain_model.plain_causal_attention(q, k3, v, window=3)
    assert torch.allclose(ow[7:], ow3[7:])
    # head h uses kv head h // (H // KVH)
    v4 = v.clone()
    v4[:, 1] += 1
    o4 = plain_model.plain_causal_attention(q, k, v4)
    assert torch.allclose(o4[:, :2], o1[:, :2]) and not torch.allclose(o4[:, 2:], o1[:, 2:])


def test_mtp_head_covers_the_right_positions(tmp_path):
    cfg, page, seed = tiny_configs.ALL["B"]
    folder = tiny_configs.make_model_folder(cfg, seed, str(tmp_path / "m"))
    c, W = plain_model.read_config(folder), plain_model.read_weights(folder)
    toks = tiny_configs.random_prompts(cfg["vocab_size"], [9], 0)[0]
    out = plain_model.plain_forward(c, W, toks)
    assert out["main"].shape == (9, cfg["vocab_size"])
    assert [m.shape[0] for m in out["mtp"]] == [8, 7]
    # a later token must not change earlier logits, and head i at p depends on token p+1+i
    toks2 = list(toks)
    toks2[5] = (toks2[5] + 1) % cfg["vocab_size"]
    out2 = plain_model.plain_forward(c, W, toks2)
    assert torch.allclose(out["main"][:5], out2["main"][:5])
    assert not torch.allclose(out["main"][5], out2["main"][5])
    assert torch.allclose(out["mtp"][0][:4], out2["mtp"][0][:4])
    assert not torch.allclose(out["mtp"][0][4], out2["mtp"][0][4])
    assert torch.allclose(out["mtp"][1][:3], out2["mtp"][1][:3])
    assert not torch.allclose(out["mtp"][1][3], out2["mtp"][1][3])


def test_plain_probs_matches_upstream_order():
    lg = torch.zeros(100)
    lg[5], lg[7] = 5.0, 4.9
    assert int(plain_model.plain_probs(lg, 1.0).argmax()) == 5
    assert int(plain_model.plain_probs(lg, 1.0, rep_penalty=2.0, ctx=[5]).argmax()) == 7
    p = plain_model.plain_probs(torch.tensor([2.0, 1.0, 0.0, -1.0]), 1.0, top_k=2)
    assert (p[2:] == 0).all() and abs(float(p.sum()) - 1) < 1e-12
    # top-p keeps the entry that crosses the line
    p = plain_model.plain_probs(torch.log(torch.tensor([0.5, 0.3, 0.15, 0.05])), 1.0, top_p=0.6)
    assert (p > 0).tolist() == [True, True, False, False]
