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
