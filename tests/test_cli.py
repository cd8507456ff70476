"""The command line, run as a user runs it: ``python -m tiny_inference_server_b200.cli`` in a
process of its own (upstream's counterpart is ``python server.py``, server.py:482-530, which has
no options; the options carry the names of its ``Request`` fields and module constants)."""
import json
import os
import subprocess
import sys

import pytest

import plain_model
import tiny_configs

ROOT = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), os.pardir))


def _cli(*args, env=None):
    e = dict(os.environ)
    e["PYTHONPATH"] = ROOT + os.pathsep + e.get("PYTHONPATH", "")
    e.update(env or {})
    return subprocess.run([sys.executable, "-m", "tiny_inference_server_b200.cli", *map(str, args)], cwd=ROOT, env=e,
                          capture_output=True, text=True, timeout=900)


def _ids(p):
    return ",".join(map(str, p))


# ---- without a GPU ------------------------------------------------------------------------------

def test_write_model_makes_a_loadable_folder(tmp_path):
    cfg_path = tmp_path / "cfg.json"
    cfg_path.write_text(json.dumps(tiny_configs.TINY_B))
    out = tmp_path / "model"
    r = _cli("--random", cfg_path, "--seed", 3, "--write-model", out)
    assert r.returncode == 0, r.stderr
    assert (out / "config.json").is_file() and (out / "model.safetensors").is_file()
    c = plain_model.read_config(str(out))
    W = plain_model.read_weights(str(out))
    assert c["hidden_size"] == tiny_configs.TINY_B["hidden_size"]
    assert W["lm_head.weight"].shape == (tiny_configs.TINY_B["vocab_size"], tiny_configs.TINY_B["hidden_size"])
    # the same seed gives the same weights as the Python entry of the random-weights mode
    again = tiny_configs.make_model_folder(tiny_configs.TINY_B, 3, str(tmp_path / "again"))
    W2 = plain_model.read_weights(again)
    assert all(bool((W[k] == W2[k]).all()) for k in W)


def test_bad_configuration_is_one_line(tmp_path):
    bad = dict(tiny_configs.TINY_A, num_kv_heads=3, colour="blue")
    bad.pop("ffn_hidden")
    cfg_path = tmp_path / "cfg.json"
    cfg_path.write_text(json.dumps(bad))
    r = _cli("--random", cfg_path, "--write-model", tmp_path / "m")
    assert r.returncode == 2
    assert "Traceback" not in r.stderr
    assert "ffn_hidden" in r.stderr and "colour" in r.stderr


def test_without_a_gpu_the_error_is_the_engines_own(tmp_path):
    folder = tiny_configs.make_model_folder(tiny_configs.TINY_A, 0, str(tmp_path / "m"))
    r = _cli("--model", folder, "--prompt-ids", "1,2,3", "--greedy", env={"CUDA_VISIBLE_DEVICES": ""})
    assert r.returncode == 2
    assert "Traceback" not in r.stderr
    assert "no CUDA device" in r.stderr and "no" in r.stderr.splitlines()[-1]


def test_no_prompt_is_a_usage_error(tmp_path):
    folder = tiny_configs.make_model_folder(tiny_configs.TINY_A, 0, str(tmp_path / "m"))
    r = _cli("--model", folder)
    assert r.returncode == 2 and "no prompt" in r.stderr


# ---- on the GPU -----------------------------------------------------------------------------------

@pytest.mark.gpu
@pytest.mark.parametrize("name,lengths,new", [("A", [1, 7, 16, 33], 12), ("B", [2, 9, 31, 64], 10)])
def test_greedy_generation_through_the_command_line(name, lengths, new, tmp_path):
    cfg, page, seed = tiny_configs.ALL[name]
    folder = tiny_configs.make_model_folder(cfg, seed, str(tmp_path / "m"))
    c, W = plain_model.read_config(folder), plain_model.read_weights(folder)
    prompts = tiny_configs.random_prompts(cfg["vocab_size"], lengths, seed=21)
    want = [plain_model.plain_greedy(c, W, p, new) for p in prompts]
    args = ["--model", folder, "--greedy", "--ignore-eos", "--dtype", "float32", "--max-new-tokens", new,
            "--tokens-per-block", page, "--json"]
    for p in prompts[:-1]:
        args += ["--prompt-ids", _ids(p)]
    pf = tmp_path / "prompts.txt"
    pf.write_text(" ".join(map(str, prompts[-1])) + "\n")
    args += ["--prompt-file", pf]
    r = _cli(*args)
    assert r.returncode == 0, r.stderr
    out = json.loads(r.stdout.strip().splitlines()[-1])
    assert out["outputs"] == want
    assert out["new_tokens"] == new * len(prompts) and out["stats"]["active"] == 0 and out["stats"]["queued"] == 0

    # a token budget of five: prompts are cut into portions beside decoding requests
    r = _cli(*args, "--max-tokens-per-step", 5, "--max-batch", 3)
    assert r.returncode == 0, r.stderr
    out = json.loads(r.stdout.strip().splitlines()[-1])
    assert out["outputs"] == want and out["stats"]["steps"] > sum(lengths) // 5

    # so few pages that the scheduler preempts and recomputes: four prompts of a page less a token each, a pool
    # that holds what they need now but not what they grow to, admission on current need
    prompts = tiny_configs.random_prompts(cfg["vocab_size"], [page - 1] * 4, seed=22)
    want = [plain_model.plain_greedy(c, W, p, new) for p in prompts]
    args = ["--model", folder, "--greedy", "--ignore-eos", "--dtype", "float32", "--max-new-tokens", new,
            "--tokens-per-block", page, "--json", "--num-pages", 4 + (new + page - 1) // page, "--plan", "cur",
            "--max-batch", 4, "--max-tokens-per-step", 16]
    for p in prompts:
        args += ["--prompt-ids", _ids(p)]
    r = _cli(*args)
    assert r.returncode == 0, r.stderr
    out = json.loads(r.stdout.strip().splitlines()[-1])
    assert out["outputs"] == want
    assert out["stats"]["preempts"] > 0 and out["stats"]["replays"] > 0 and out["stats"]["min_free_pages"] == 0


@pytest.mark.gpu
def test_random_model_and_text_output_through_the_command_line(tmp_path):
    cfg_path = tmp_path / "cfg.json"
    cfg_path.write_text(json.dumps(tiny_configs.TINY_A))
    folder = tiny_configs.make_model_folder(tiny_configs.TINY_A, 9, str(tmp_path / "m"))
    c, W = plain_model.read_config(folder), plain_model.read_weights(folder)
    prompt = [5, 17, 3, 200]
    want = plain_model.plain_greedy(c, W, prompt, 8)
    r = _cli("--random", cfg_path, "--seed", 9, "--prompt-ids", "5 17 3 200", "--temperature", 0, "--ignore-eos",
             "--dtype", "fp32", "--max-new-tokens", 8, "--mtp")
    assert r.returncode == 0, r.stderr
    lines = r.stdout.splitlines()
    assert "PROMPT: 5 17 3 200" in lines
    assert "OUTPUT: " + " ".join(map(str, want)) in lines
    # sampling options with upstream's names; the same seed gives the same tokens
    a = _cli("--model", folder, "--prompt-ids", _ids(prompt), "--temperature", 0.9, "--top-k", 20, "--top-p", 0.9,
             "--rep-penalty", 1.2, "--seed", 4, "--max-new-tokens", 6, "--ignore-eos", "--json")
    b = _cli("--model", folder, "--prompt-ids", _ids(prompt), "--temperature", 0.9, "--top-k", 20, "--top-p", 0.9,
             "--rep-penalty", 1.2, "--seed", 4, "--max-new-tokens", 6, "--ignore-eos", "--json", "--no-cuda-graphs")
    assert a.returncode == 0 and b.returncode == 0, a.stderr + b.stderr
    assert json.loads(a.stdout.strip().splitlines()[-1])["outputs"] == \
        json.loads(b.stdout.strip().splitlines()[-1])["outputs"]
