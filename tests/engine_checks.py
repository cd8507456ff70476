"""Checks shared by the CPU and the GPU tests of the ``Engine``."""
from __future__ import annotations

import plain_model
import tiny_configs


def check_mtp_logits_through_engine(make_engine, name, tmp_path, tol, *, lengths=(3, 11, 20, 6), new=14,
                                    engine_kw=None, pipeline=True, expect_preemption=False):
    """Generate greedily with the MTP heads running beside the trunk and compare, at every step, the
    main logits and every valid MTP logit that the step emits with the plain implementation on the
    request's final sequence.  The step that feeds the token at position p emits main logits for p
    and head i's logits for position p-1-i (valid when that is not negative); under preemption a
    request's prompt and its generated tokens are fed again and must give the same logits again."""
    import torch
    from tiny_inference_server_b200.api import SamplingParams

    cfg, page, seed = tiny_configs.ALL[name]
    folder = tiny_configs.make_model_folder(cfg, seed, str(tmp_path / f"mtp{name}"))
    c, W = plain_model.read_config(folder), plain_model.read_weights(folder)
    prompts = tiny_configs.random_prompts(cfg["vocab_size"], list(lengths), seed=13)
    eng = make_engine(folder, page, mtp=True, **(engine_kw or {}))
    eng.pipeline = pipeline
    seen = []                # (request, position of the wanted row, main logits, [(head logits, valid)])

    def listen(entries, out):
        j = 0
        for req, start, n in entries:
            sampled = start + n == len(req.ids)          # the portion reaches the request's last token
            if not sampled:
                continue
            aux = [(out.aux[i][j].detach().float().cpu(), bool(out.aux_valid[i][j])) for i in range(len(out.aux))]
            seen.append((req, start + n - 1, out.main[j].detach().float().cpu(), aux))
            j += 1
        assert j == out.main.shape[0]

    eng.step_listener = listen
    reqs = [eng.submit(p, SamplingParams(max_new_tokens=new, temperature=0.0, ignore_eos=True)) for p in prompts]
    eng.run()
    eng.runner.cache.check()
    assert eng.runner.cache.drained()
    plain = {id(r): plain_model.plain_forward(c, W, r.ids) for r in reqs}
    n_heads = cfg["num_mtp_heads"]
    checked = [0] * (1 + n_heads)
    worst = 0.0
    for req, pos, main, aux in seen:
        ref = plain[id(req)]
        err = float((main.double() - ref["main"][pos]).abs().max())
        assert err < tol, f"main logits of request {req.id} at position {pos}: {err}"
        checked[0] += 1
        assert len(aux) == n_heads
        for i, (lg, valid) in enumerate(aux):
            hp = pos - 1 - i
            assert valid == (hp >= 0), f"head {i} at position {pos}: valid={valid}"
            if valid:
                err = float((lg.double() - ref["mtp"][i][hp]).abs().max())
                assert err < tol, f"mtp head {i} of request {req.id} for position {hp}: {err}"
                worst = max(worst, err)
                checked[1 + i] += 1
    assert all(k >= len(prompts) * (new - 2) for k in checked), checked
    if expect_preemption:
        assert eng.scheduler.preempts > 0 and eng.scheduler.replays > 0
    # the tokens are the plain implementation's too (float32 only: bfloat16 may pick another near-tie)
    return eng, reqs, worst
