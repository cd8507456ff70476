"""Configuration, registry, weight loading errors and the random-weights mode (CPU)."""
import json
import os

import pytest
import torch

import tiny_configs
from tiny_inference_server_b200 import ConfigError, GqaMtpConfig, build_model, config_from_dict, config_from_folder
from tiny_inference_server_b200.registry import architectures
from tiny_inference_server_b200.weights import WeightError, load_weights, random_tensors, write_random_model


def test_architecture_is_chosen_by_name():
    assert "gqa_mtp_transformer" in architectures()
    cfg = config_from_dict(dict(tiny_configs.TINY_A))
    assert isinstance(cfg, GqaMtpConfig) and cfg.group_size == 2 and cfg.head_dim == 16
    with pytest.raises(ConfigError, match="unknown architecture"):
        config_from_dict(dict(tiny_configs.TINY_A, architecture="nope"))


def test_upstream_field_names_are_aliases():
    # Config/config.py:11-23 of the upstream project: its 0.9B model
    cfg = config_from_dict(dict(D_MODEL=1536, VOCAB_SIZE=48011, MAX_CONTEXT=8192, MAX_FREQ=10000, N_HEAD=12,
                                NUM_LAYERS=30, FFN_HIDDEN_DIM=4096, NUM_GROUPS=4, MTP_HEADS=2))
    assert (cfg.hidden_size, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim) == (1536, 12, 3, 128)
    assert cfg.rms_norm_eps == 2e-8 and cfg.rope_theta == 10000 and cfg.num_mtp_heads == 2
    assert cfg.tie_word_embeddings


def test_config_errors_name_every_problem():
    with pytest.raises(ConfigError) as e:
        config_from_dict(dict(architecture="gqa_mtp_transformer", vocab_size=10, hidden_size=8, bogus=1, extra=2))
    msg = str(e.value)
    for word in ("num_layers", "num_heads", "num_kv_heads", "ffn_hidden", "bogus", "extra"):
        assert word in msg
    base = dict(tiny_configs.TINY_A)
    with pytest.raises(ConfigError, match="not a multiple"):
        config_from_dict(dict(base, num_kv_heads=3))
    with pytest.raises(ConfigError, match="even"):
        config_from_dict(dict(base, head_dim=15))
    with pytest.raises(ConfigError, match="cache_source"):
        config_from_dict(dict(base, cache_source=[None]))
    with pytest.raises(ConfigError, match="earlier"):
        config_from_dict(dict(base, cache_source=[1, None]))
    with pytest.raises(ConfigError, match="layer_order"):
        config_from_dict(dict(base, layer_order=[0, 5]))


def test_a_layer_may_not_see_further_back_than_the_cache_it_reads():
    """Pages of a windowed layer's cache are given back as the window passes them; a layer that reads
    that cache must not reach behind the window."""
    base = dict(tiny_configs.TINY_A, num_layers=3, num_mtp_heads=0, layer_order=[0, 1, 2])
    # layer 2 reads the cache of layer 1; both windowed: fine
    config_from_dict(dict(base, sliding_window=8, cache_source=[None, None, 1]))
    # both unwindowed, and a windowed reader of a full cache: fine
    config_from_dict(dict(base, cache_source=[None, None, 1]))
    config_from_dict(dict(base, sliding_window=8, full_attention_layers=[1], cache_source=[None, None, 1]))
    # a full-attention reader of a windowed cache: refused, with both layers named
    with pytest.raises(ConfigError, match=r"layer 2 sees every key but layer 1.*keeps only 8"):
        config_from_dict(dict(base, sliding_window=8, full_attention_layers=[2], cache_source=[None, None, 1]))


def test_config_json_round_trip(tmp_path):
    cfg = config_from_dict(dict(tiny_configs.TINY_C))
    folder = write_random_model(str(tmp_path / "m"), cfg, seed=3)
    again = config_from_folder(folder)
    assert again.to_dict() == cfg.to_dict()
    with pytest.raises(ConfigError, match="no config.json"):
        config_from_folder(str(tmp_path / "missing"))


def test_no_size_in_code_every_shape_follows_the_config():
    a = build_model(config_from_dict(dict(tiny_configs.TINY_A))).expected_tensors()
    b = build_model(config_from_dict(dict(tiny_configs.TINY_B))).expected_tensors()
    assert a["embedding.weight"].shape == (256, 64) and b["embedding.weight"].shape == (512, 128)
    assert a["transformer_block_list.1.att.kv_proj.weight"].shape == (64, 2 * 2 * 16)
    assert b["transformer_block_list.2.att.kv_proj.weight"].shape == (128, 2 * 1 * 32)
    assert b["mtp_heads_list.1.proj.weight"].shape == (256, 128)
    assert "lm_head.weight" in b and "lm_head.weight" not in a
    assert "mtp_heads_list.1.proj.weight" not in a
    # upstream's tensor names (main_models_new.py named_parameters)
    for name in ("transformer_block_list.0.att.q_proj.weight", "transformer_block_list.0.att.rms_norm_att.scale",
                 "transformer_block_list.0.att.linear_proj.weight", "transformer_block_list.0.ffn.swig.linear1.weight",
                 "transformer_block_list.0.ffn.swig.linear2.weight", "transformer_block_list.0.ffn.fc.weight",
                 "transformer_block_list.0.rms_norm_ffn.scale", "rms_out.scale", "mtp_heads_list.0.rms_embed.scale",
                 "mtp_heads_list.0.rms_out.scale", "mtp_heads_list.0.trans_block.att.q_proj.weight"):
        assert name in a, name


def test_random_weights_are_reproducible_and_bfloat16(tmp_path):
    from safetensors.torch import load_file
    cfg = config_from_dict(dict(tiny_configs.TINY_A))
    f1 = write_random_model(str(tmp_path / "a"), cfg, seed=5)
    f2 = write_random_model(str(tmp_path / "b"), cfg, seed=5)
    f3 = write_random_model(str(tmp_path / "c"), cfg, seed=6)
    w1, w2, w3 = (load_file(os.path.join(f, "model.safetensors")) for f in (f1, f2, f3))
    assert all(torch.equal(w1[k], w2[k]) for k in w1)
    assert any(not torch.equal(w1[k], w3[k]) for k in w1)
    assert all(t.dtype == torch.bfloat16 for t in w1.values())
    assert abs(float(w1["rms_out.scale"].float().mean()) - 1.0) < 0.05
    assert abs(float(w1["embedding.weight"].float().std()) - 0.02) < 0.005
    assert sorted(os.listdir(f1)) == ["config.json", "model.safetensors"]


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    from safetensors.torch import load_file, save_file
    cfg = config_from_dict(dict(tiny_configs.TINY_A))
    folder = write_random_model(str(tmp_path / "m"), cfg, seed=0)
    path = os.path.join(folder, "model.safetensors")
    w = load_file(path)
    del w["rms_out.scale"]
    del w["transformer_block_list.1.ffn.fc.weight"]
    w["lm_head.weight"] = torch.zeros(256, 64, dtype=torch.bfloat16)        # tied model: not expected
    w["stray.tensor"] = torch.zeros(3)
    w["embedding.weight"] = torch.zeros(255, 64, dtype=torch.bfloat16)
    save_file(w, path)
    expected = build_model(cfg).expected_tensors()
    with pytest.raises(WeightError) as e:
        load_weights(folder, expected)
    msg = str(e.value)
    assert "missing (2)" in msg and "rms_out.scale" in msg and "transformer_block_list.1.ffn.fc.weight" in msg
    assert "unexpected (2)" in msg and "lm_head.weight" in msg and "stray.tensor" in msg
    assert "wrong shape (1)" in msg and "(255, 64)" in msg and "(256, 64)" in msg


def test_stored_dtypes_are_kept(tmp_path):
    from safetensors.torch import load_file, save_file
    cfg = config_from_dict(dict(tiny_configs.TINY_A))
    folder = write_random_model(str(tmp_path / "m"), cfg, seed=0)
    path = os.path.join(folder, "model.safetensors")
    w = load_file(path)
    w["rms_out.scale"] = w["rms_out.scale"].to(torch.float32)
    w["transformer_block_list.0.rms_norm_ffn.scale"] = w["transformer_block_list.0.rms_norm_ffn.scale"].to(torch.float16)
    save_file(w, path)
    got = load_weights(folder, build_model(cfg).expected_tensors())
    assert got["rms_out.scale"].dtype == torch.float32                       # stored in 32-bit: stays so
    assert got["embedding.weight"].dtype == torch.bfloat16                   # kept in bfloat16
    assert got["transformer_block_list.0.rms_norm_ffn.scale"].dtype == torch.float32
    with pytest.raises(WeightError, match="no \\*.safetensors"):
        load_weights(str(tmp_path), {})
