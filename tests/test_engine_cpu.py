"""Generation through the Python entry point on the CPU (plain references in place of the
kernels): greedy tokens equal the plain implementation's, with chunked prompts, a small
pool that forces preemption, and pages all given back."""
import pytest

import plain_model
import tiny_configs
from tiny_inference_server_b200.api import Engine, SamplingParams
from tiny_inference_server_b200.config import EngineConfig


def _engine(folder, page, **kw):
    base = dict(dtype="float32", page_size=page, num_pages=64, max_batch=4, max_tokens_per_step=2048,
                device="cpu", cuda_graphs=False)
    base.update(kw)
    return Engine.from_folder(folder, EngineConfig(**base))


@pytest.mark.parametrize("name,lengths,new", [("A", [1, 7, 16, 33], 12), ("B", [2, 9, 31, 64], 10)])
def test_greedy_equals_plain(name, lengths, new, tmp_path, ref_ops):
    cfg, page, seed = tiny_configs.ALL[name]
    folder = tiny_configs.make_model_folder(cfg, seed, str(tmp_path / "m"))
    c, W = plain_model.read_config(folder), plain_model.read_weights(folder)
    prompts = tiny_configs.random_prompts(cfg["vocab_size"], lengths, seed=7)
    want = [plain_model.plain_greedy(c, W, p, new) for p in prompts]
    sp = SamplingParams(max_new_tokens=new, temperature=0.0, ignore_eos=True)

    eng = _engine(folder, page)
    assert eng.generate(prompts, sp) == want
    assert eng.runner.cache.drained()

    # prompts cut into small portions, mixed with decoding requests
    eng = _engine(folder, page, max_tokens_per_step=5, max_batch=3)
    assert eng.generate(prompts, sp) == want
    assert eng.runner.cache.drained()

    # so few pages that requests are preempted and replayed: four prompts of one page each
    # minus a token, a pool of five pages, admission on current need
    prompts = tiny_configs.random_prompts(cfg["vocab_size"], [page - 1] * 4, seed=8)
    want = [plain_model.plain_greedy(c, W, p, new) for p in prompts]
    eng = _engine(folder, page, num_pages=5, admission="cur", max_batch=4, max_tokens_per_step=16)
    assert eng.generate(prompts, sp) == want
    assert eng.scheduler.preempts > 0 and eng.scheduler.replays > 0
    eng.runner.cache.check()
    assert eng.runner.cache.drained()


@pytest.mark.parametrize("name", ["A", "B"])
def test_step_in_flight_changes_nothing(name, tmp_path, ref_ops):
    """With one step kept in flight the tokens are those of the step-by-step engine, also when
    requests end at different steps, on the end-of-sequence token (noticed a step late) or on
    their length, and when pages are short."""
    cfg, page, seed = tiny_configs.ALL[name]
    folder = tiny_configs.make_model_folder(cfg, seed, str(tmp_path / "m"))
    c, W = plain_model.read_config(folder), plain_model.read_weights(folder)
    prompts = tiny_configs.random_prompts(cfg["vocab_size"], [3, 11, 20, 6], seed=11)
    full = [plain_model.plain_greedy(c, W, p, 14) for p in prompts]
    news = [14, 9, 12, 5]
    sps = [SamplingParams(max_new_tokens=n, temperature=0.0, ignore_eos=True) for n in news]
    want = [f[:n] for f, n in zip(full, news)]
    for pipeline in (False, True):
        eng = _engine(folder, page)
        eng.pipeline = pipeline
        assert eng.generate(prompts, sps) == want
        assert (eng.steps_behind > 0) == pipeline
        assert eng.runner.cache.drained()
        eng.runner.cache.check()

    # the end-of-sequence token: the seventh token of the first request
    eos = full[0][6]
    want = [f[: f.index(eos) + 1] if eos in f else f for f in full]
    sp = SamplingParams(max_new_tokens=14, temperature=0.0)
    for pipeline in (False, True):
        eng = _engine(folder, page)
        eng.pipeline = pipeline
        eng.scheduler.eos_token_id = eos
        assert eng.generate(prompts, sp) == want
        assert eng.runner.cache.drained()
        eng.runner.cache.check()

    # short of pages while a step is in flight: the engine falls back to deciding step by step
    prompts = tiny_configs.random_prompts(cfg["vocab_size"], [page - 1] * 4, seed=8)
    want = [plain_model.plain_greedy(c, W, p, 12) for p in prompts]
    eng = _engine(folder, page, num_pages=6, admission="cur", max_tokens_per_step=64)
    assert eng.generate(prompts, SamplingParams(max_new_tokens=12, temperature=0.0, ignore_eos=True)) == want
    assert eng.scheduler.preempts > 0 and eng.steps_behind > 0
    assert eng.runner.cache.drained()


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("how", ["plain", "chunked", "preempted", "step_by_step"])
def test_mtp_heads_beside_the_trunk_through_the_engine(name, how, tmp_path, ref_ops):
    """``EngineConfig.mtp``: every step also runs the MTP heads; their logits equal the plain
    implementation's under chunked prompts, preemption with recomputation, and the step in flight."""
    import engine_checks
    cfg, page, _ = tiny_configs.ALL[name]
    kw = {"plain": {}, "step_by_step": {},
          "chunked": dict(max_tokens_per_step=5, max_batch=3),
          "preempted": dict(num_pages=5 if name == "A" else 9, admission="cur", max_tokens_per_step=16)}[how]
    lengths = [page - 1] * 4 if how == "preempted" else (3, 11, 20, 6)
    eng, reqs, _ = engine_checks.check_mtp_logits_through_engine(
        _engine, name, tmp_path, 2e-4, lengths=lengths, new=12, engine_kw=kw, pipeline=how != "step_by_step",
        expect_preemption=how == "preempted")
    c, W = plain_model.read_config(str(tmp_path / f"mtp{name}")), plain_model.read_weights(str(tmp_path / f"mtp{name}"))
    for r in reqs:
        assert r.out_ids() == plain_model.plain_greedy(c, W, r.ids[:r.prompt_len], 12)
    assert (eng.steps_behind > 0) == (how != "step_by_step")


@pytest.mark.parametrize("seed", range(12))
def test_random_workloads_equal_plain(seed, tmp_path, ref_ops):
    """Workloads drawn at random — number and lengths of prompts, tokens to generate, an
    end-of-sequence token, pool size down to what one request needs, batch limit, token budget,
    admission plan, with and without a step in flight: the tokens equal the plain implementation's
    and every page comes back."""
    import random
    rng = random.Random(seed)
    name = rng.choice(["A", "B", "D"])
    cfg, page, mseed = tiny_configs.ALL[name]
    folder = tiny_configs.make_model_folder(cfg, mseed, str(tmp_path / "m"))
    c, W = plain_model.read_config(folder), plain_model.read_weights(folder)
    nreq = rng.randint(1, 6)
    lengths = [rng.randint(1, 40) for _ in range(nreq)]
    prompts = tiny_configs.random_prompts(cfg["vocab_size"], lengths, seed=seed)
    news = [rng.randint(1, 14) for _ in range(nreq)]
    full = [plain_model.plain_greedy(c, W, p, n) for p, n in zip(prompts, news)]
    use_eos = rng.random() < 0.5
    eos = rng.choice(full[0]) if use_eos else None
    want = [(f[: f.index(eos) + 1] if (eos is not None and eos in f) else f) for f in full]
    max_need = max((l + n + page) // page + 1 for l, n in zip(lengths, news))
    eng = _engine(folder, page, num_pages=rng.randint(max_need, max_need * nreq + 2), max_batch=rng.randint(1, 5),
                  max_tokens_per_step=rng.choice([3, 7, 16, 64, 2048]), admission=rng.choice(["final", "cur"]))
    eng.pipeline = rng.random() < 0.7
    eng.scheduler.eos_token_id = eos
    sps = [SamplingParams(max_new_tokens=n, temperature=0.0, ignore_eos=not use_eos) for n in news]
    assert eng.generate(prompts, sps) == want
    eng.runner.cache.check()
    assert eng.runner.cache.drained()
