"""The converter from upstream's positional checkpoint lists to a model folder (CPU).  Where a checkout
of the upstream project is at hand, its own ``named_parameters()``, its own checkpoint format and its
own dense oracle are used; otherwise only the converter's own bookkeeping is checked."""
import json
import os
import sys

import numpy as np
import pytest
import torch

import plain_model
import tiny_configs
from tiny_inference_server_b200 import config_from_dict
from tiny_inference_server_b200.weights import WeightError
from tiny_inference_server_b200.weights.convert_upstream import convert, main, split_names, upstream_parameter_names

ROOT = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), os.pardir))
CFG = dict(D_MODEL=64, VOCAB_SIZE=120, MAX_CONTEXT=64, MAX_FREQ=10000, N_HEAD=4, NUM_LAYERS=2, FFN_HIDDEN_DIM=96,
           NUM_GROUPS=2, MTP_HEADS=2)


def _upstream():
    for folder in (os.environ.get("TIS_UPSTREAM"), "/root/reference", os.path.join(ROOT, "baseline", "_ref")):
        if folder and os.path.isfile(os.path.join(folder, "main_models_new.py")):
            if folder not in sys.path:
                sys.path.insert(0, folder)
            import main_models_new
            return folder, main_models_new
    pytest.skip("no checkout of the upstream project")


def test_names_and_split_follow_the_configuration():
    cfg = config_from_dict(dict(CFG))
    names = upstream_parameter_names(cfg.num_layers, cfg.num_mtp_heads)
    assert len(names) == 1 + 8 * 2 + 1 + 2 * (3 + 8) and len(set(names)) == len(names)
    from tiny_inference_server_b200 import build_model
    shapes = {n: tuple(s.shape) for n, s in build_model(cfg).expected_tensors().items()}
    two, one = split_names(names, shapes)
    assert "embedding.weight" in one and "mtp_heads_list.0.rms_embed.scale" in one
    assert all(len(shapes[n]) == 2 for n in two) and len(two) + len(one) == len(names)
    # a checkpoint that does not fit: every problem named
    ckpt = {"master_2d": [torch.zeros(shapes[n]) for n in two], "master_1d": [torch.zeros(shapes[n]) for n in one]}
    ckpt["master_2d"][3] = torch.zeros(5, 5)
    with pytest.raises(WeightError, match=two[3].replace(".", r"\.")):
        convert(ckpt, cfg)
    with pytest.raises(WeightError, match="master_1d holds"):
        convert({"master_2d": ckpt["master_2d"], "master_1d": ckpt["master_1d"][:4]}, cfg)


def test_order_is_upstreams_own_and_logits_survive_the_conversion(tmp_path):
    folder, M = _upstream()
    cfg = config_from_dict(dict(CFG))
    torch.manual_seed(3)
    group = cfg.num_heads // cfg.num_kv_heads
    m = M.Transformer(cfg.vocab_size, cfg.max_context, cfg.rope_theta, cfg.hidden_size, cfg.num_heads, cfg.num_layers,
                      cfg.ffn_hidden, group, mtp_heads=cfg.num_mtp_heads).eval()
    assert [n for n, _ in m.named_parameters()] == upstream_parameter_names(cfg.num_layers, cfg.num_mtp_heads)
    # a checkpoint as upstream's training writes it (main_models_new.py:238-239 in reverse)
    ckpt = {"master_2d": [p.detach().clone() for n, p in m.named_parameters() if p.ndim == 2 and "embed" not in n],
            "master_1d": [p.detach().clone() for n, p in m.named_parameters() if p.ndim == 1 or "embed" in n],
            "opt_step": 7}
    torch.save(ckpt, tmp_path / "ckpt.pt")
    (tmp_path / "cfg.json").write_text(json.dumps(CFG))
    assert main([str(tmp_path / "ckpt.pt"), "--config", str(tmp_path / "cfg.json"), "--out", str(tmp_path / "m"),
                 "--dtype", "float32"]) == 0
    c, W = plain_model.read_config(str(tmp_path / "m")), plain_model.read_weights(str(tmp_path / "m"))
    for n, p in m.named_parameters():
        assert torch.equal(W[n].float(), p.detach().float()), n
    # the logits of upstream's own dense oracle on its own model equal the plain implementation on the folder
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    import make_golden
    toks = [5, 100, 17, 3, 99, 50, 0, 42, 42, 7]
    dense = make_golden.upstream_dense_forward(folder, M, dict(hidden_size=cfg.hidden_size, num_heads=cfg.num_heads,
                                                               num_kv_heads=cfg.num_kv_heads))(m, torch.tensor(toks))
    ours = plain_model.plain_forward(c, W, toks, mtp=False)["main"]
    np.testing.assert_allclose(ours.numpy(), dense.detach().numpy(), rtol=0, atol=5e-6)
    # fewer MTP heads than were trained: a prefix of both lists
    fewer = config_from_dict(dict(CFG, MTP_HEADS=1))
    t = convert(ckpt, fewer, torch.float32)
    assert "mtp_heads_list.0.proj.weight" in t and "mtp_heads_list.1.proj.weight" not in t
    assert torch.equal(t["mtp_heads_list.0.trans_block.ffn.fc.weight"],
                       dict(m.named_parameters())["mtp_heads_list.0.trans_block.ffn.fc.weight"].detach())
