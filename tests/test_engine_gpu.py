"""Generation through the Python entry point on the GPU, long decoding, the first tokens
of a sequence, each part alone, and a toy mixer with state of its own that is registered,
built and stepped without any change to the engine's files."""
import math
import os

import pytest
import torch

import plain_model
import tiny_configs

pytestmark = pytest.mark.gpu


def _engine(folder, page, **kw):
    from tiny_inference_server_b200.api import Engine
    from tiny_inference_server_b200.config import EngineConfig
    base = dict(dtype="float32", page_size=page, num_pages=128, max_batch=4, max_tokens_per_step=2048)
    base.update(kw)
    return Engine.from_folder(folder, EngineConfig(**base))


def _model(name, tmp_path):
    cfg, page, seed = tiny_configs.ALL[name]
    folder = tiny_configs.make_model_folder(cfg, seed, str(tmp_path / f"m{name}"))
    return cfg, page, folder, plain_model.read_config(folder), plain_model.read_weights(folder)


@pytest.mark.parametrize("name,lengths,new", [("A", [1, 7, 16, 33], 24), ("B", [2, 9, 31, 64, 100, 130], 40)])
def test_greedy_generation_equals_plain_float32(name, lengths, new, tmp_path):
    from tiny_inference_server_b200.api import SamplingParams
    cfg, page, folder, c, W = _model(name, tmp_path)
    prompts = tiny_configs.random_prompts(cfg["vocab_size"], lengths, seed=7)
    want = [plain_model.plain_greedy(c, W, p, new) for p in prompts]
    sp = SamplingParams(max_new_tokens=new, temperature=0.0, ignore_eos=True)
    eng = _engine(folder, page, max_batch=8)
    assert eng.generate(prompts, sp) == want
    assert eng.runner.cache.drained()
    # one mixed batch with chunked prefill, as few tokens a step as 5
    eng = _engine(folder, page, max_tokens_per_step=5, max_batch=6)
    assert eng.generate(prompts, sp) == want
    # upstream's greedy setting: top_k=1 at temperature 1 (test_server.py:110)
    eng = _engine(folder, page, max_batch=8)
    assert eng.generate(prompts, SamplingParams(max_new_tokens=new, temperature=1.0, top_k=1, ignore_eos=True)) == want


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("graphs", [True, False])
def test_step_in_flight_float32(name, graphs, tmp_path):
    """One decode step kept in flight (tokens fed on the device, read back a step late): the
    same tokens as step by step and as the plain implementation; requests of different
    lengths, the end-of-sequence token, sampling with a seed."""
    from tiny_inference_server_b200.api import SamplingParams
    cfg, page, folder, c, W = _model(name, tmp_path)
    prompts = tiny_configs.random_prompts(cfg["vocab_size"], [3, 11, 20, 6, 40], seed=11)
    full = [plain_model.plain_greedy(c, W, p, 30) for p in prompts]
    news = [30, 9, 22, 5, 17]
    sps = [SamplingParams(max_new_tokens=n, temperature=0.0, ignore_eos=True) for n in news]
    eng = _engine(folder, page, max_batch=8, cuda_graphs=graphs)
    assert eng.generate(prompts, sps) == [f[:n] for f, n in zip(full, news)]
    assert eng.steps_behind > 10 and eng.runner.cache.drained()

    eos = full[0][12]
    want = [f[: f.index(eos) + 1] if eos in f else f for f in full]
    eng = _engine(folder, page, max_batch=8, cuda_graphs=graphs)
    eng.scheduler.eos_token_id = eos
    assert eng.generate(prompts, SamplingParams(max_new_tokens=30, temperature=0.0)) == want
    assert eng.steps_behind > 5 and eng.runner.cache.drained()
    eng.runner.cache.check()

    # drawn tokens: the same seed gives the same tokens with and without the step in flight
    sp = SamplingParams(max_new_tokens=20, temperature=0.9, top_k=12, top_p=0.95, rep_penalty=1.2, seed=5,
                        ignore_eos=True)
    outs = []
    for pipeline in (True, False):
        eng = _engine(folder, page, max_batch=8, cuda_graphs=graphs)
        eng.pipeline = pipeline
        outs.append(eng.generate(prompts, sp))
    assert outs[0] == outs[1]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("name,how", [("A", "plain"), ("A", "chunked"), ("A", "preempted"), ("B", "plain"),
                                      ("B", "chunked"), ("B", "preempted"), ("B", "step_by_step")])
def test_mtp_heads_beside_the_trunk_through_the_engine(name, how, graphs, dtype, tmp_path):
    """``EngineConfig.mtp``: the MTP heads run in every step of generation, inside the decode graph and
    the step kept in flight (where the head's input reads tokens fed on the device); their logits equal
    the plain implementation's under chunked prompts and under preemption with recomputation (upstream
    checks its heads by speculative decoding giving the tokens of plain decoding, test_server.py:104-118)."""
    import engine_checks
    cfg, page, _ = tiny_configs.ALL[name]
    kw = {"plain": {}, "step_by_step": {},
          "chunked": dict(max_tokens_per_step=5, max_batch=3),
          "preempted": dict(num_pages=5 if name == "A" else 9, admission="cur", max_tokens_per_step=16)}[how]
    kw = dict(kw, dtype=dtype, cuda_graphs=graphs)
    lengths = [page - 1] * 4 if how == "preempted" else (3, 11, 20, 6)
    eng, reqs, worst = engine_checks.check_mtp_logits_through_engine(
        _engine, name, tmp_path, 2e-4 if dtype == "float32" else 3e-2, lengths=lengths, new=14, engine_kw=kw,
        pipeline=how != "step_by_step", expect_preemption=how == "preempted")
    assert (eng.steps_behind > 0) == (how != "step_by_step")
    if graphs:
        assert eng.runner.graphs is not None and eng.runner.graphs.replays > 5
    if dtype == "float32":
        c, W = plain_model.read_config(str(tmp_path / f"mtp{name}")), plain_model.read_weights(str(tmp_path / f"mtp{name}"))
        for r in reqs:
            assert r.out_ids() == plain_model.plain_greedy(c, W, r.ids[:r.prompt_len], 14)


def test_step_phases_are_timed_when_asked(tmp_path):
    """``EngineConfig.profile``: host and device time per phase of the steps, in ``Engine.stats()``
    (upstream's Probe, evals.py:42-83, gives admit / prefill / decode times the same way)."""
    from tiny_inference_server_b200.api import SamplingParams
    cfg, page, folder, c, W = _model("A", tmp_path)
    prompts = tiny_configs.random_prompts(cfg["vocab_size"], [9, 30], seed=3)
    eng = _engine(folder, page, profile=True)
    eng.generate(prompts, SamplingParams(max_new_tokens=12, temperature=0.0, ignore_eos=True))
    ph = eng.stats()["phases"]
    assert ph["steps"] >= 12
    assert set(ph["host_ms"]) >= {"admit", "plan", "launch", "read_back"}
    assert ph["device_ms"]["prefill"] > 0 and ph["device_ms"]["decode"] > 0
    assert ph["calls"]["device:decode"] >= 10 and ph["calls"]["device:prefill"] >= 1
    assert "phases" not in _engine(folder, page).stats()


def test_greedy_generation_with_preemption_float32(tmp_path):
    from tiny_inference_server_b200.api import SamplingParams
    cfg, page, folder, c, W = _model("A", tmp_path)
    prompts = tiny_configs.random_prompts(cfg["vocab_size"], [page - 1] * 4, seed=8)
    want = [plain_model.plain_greedy(c, W, p, 12) for p in prompts]
    eng = _engine(folder, page, num_pages=5, admission="cur", max_tokens_per_step=16)
    got = eng.generate(prompts, SamplingParams(max_new_tokens=12, temperature=0.0, ignore_eos=True))
    assert got == want and eng.scheduler.preempts > 0
    eng.runner.cache.check()
    assert eng.runner.cache.drained()


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_bfloat16_stays_on_the_plain_argmax(name, tmp_path):
    """bfloat16 rounding may pick another token where two logits are close; every token the
    engine picks must be, in the plain implementation given the same history, within a
    small margin of the best logit."""
    from tiny_inference_server_b200.api import SamplingParams
    cfg, page, folder, c, W = _model(name, tmp_path)
    prompts = tiny_configs.random_prompts(cfg["vocab_size"], [3, 20, 45], seed=9)
    eng = _engine(folder, page, dtype="bfloat16")
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=16, temperature=0.0, ignore_eos=True))
    for p, o in zip(prompts, outs):
        logits = plain_model.plain_forward(c, W, list(p) + o[:-1], mtp=False)["main"]
        for j, tok in enumerate(o):
            row = logits[len(p) - 1 + j]
            assert float(row.max() - row[tok]) < 3e-2, f"token {j}: margin {float(row.max() - row[tok])}"


def test_long_decoding_float32(tmp_path):
    """200 tokens decoded one by one after a short prompt, across many page edges."""
    from tiny_inference_server_b200.api import SamplingParams
    cfg, page, folder, c, W = _model("B", tmp_path)
    prompt = tiny_configs.random_prompts(cfg["vocab_size"], [5], seed=10)[0]
    want = plain_model.plain_greedy(c, W, prompt, 200)
    eng = _engine(folder, page)
    got = eng.generate([prompt], SamplingParams(max_new_tokens=200, temperature=0.0, ignore_eos=True))[0]
    first_bad = next((i for i, (a, b) in enumerate(zip(got, want)) if a != b), None)
    assert first_bad is None, f"first wrong token at {first_bad} (position {len(prompt) + (first_bad or 0)})"


def test_first_tokens_of_a_sequence(tmp_path):
    """Positions 0, 1, 2 fed one by one: no earlier key, one-token prompt, MTP heads not yet
    valid."""
    from tiny_inference_server_b200.config import EngineConfig
    from tiny_inference_server_b200.engine import ModelRunner, StepEntry
    cfg, page, folder, c, W = _model("B", tmp_path)
    toks = [11, 400, 3, 77]
    plain = plain_model.plain_forward(c, W, toks)
    for dtype, tol in (("float32", 2e-4), ("bfloat16", 3e-2)):
        r = ModelRunner.from_folder(folder, EngineConfig(dtype=dtype, page_size=page, num_pages=8, mtp=True))
        s = r.add_request()
        for p, t in enumerate(toks):
            out = r.step([StepEntry(s, [t], [0])])
            assert float((out.main[0].cpu() - plain["main"][p]).abs().max()) < tol
            for i in range(cfg["num_mtp_heads"]):
                valid = bool(out.aux_valid[i][0])
                assert valid == (p - 1 - i >= 0)
                if valid:
                    assert float((out.aux[i][0].cpu() - plain["mtp"][i][p - 1 - i]).abs().max()) < tol
        r.check_fault()


def test_temperature_sampling_is_reproducible_and_batch_independent(tmp_path):
    from tiny_inference_server_b200.api import SamplingParams
    cfg, page, folder, c, W = _model("A", tmp_path)
    prompts = tiny_configs.random_prompts(cfg["vocab_size"], [4, 9, 17], seed=11)
    sp = [SamplingParams(max_new_tokens=10, temperature=0.9, top_k=50, top_p=0.95, rep_penalty=1.1, seed=100 + i,
                         ignore_eos=True) for i in range(3)]
    a = _engine(folder, page).generate(prompts, sp)
    b = _engine(folder, page).generate(prompts, sp)
    assert a == b
    alone = [_engine(folder, page).generate([p], [s])[0] for p, s in zip(prompts, sp)]
    assert alone == a
    other = _engine(folder, page).generate(prompts, [SamplingParams(max_new_tokens=10, temperature=0.9, seed=7 + i,
                                                                    ignore_eos=True) for i in range(3)])
    assert other != a


# ----------------------------------------------------------------------------------------
# each part alone
# ----------------------------------------------------------------------------------------

def _ctx(dtype):
    from tiny_inference_server_b200.parts import BuildContext
    return BuildContext(torch.device("cuda:0"), dtype)


def _random_part_weights(part, dtype, seed):
    from tiny_inference_server_b200.weights import random_tensors
    specs = {}
    for p in part.walk():
        specs.update(p.expected_tensors())
    return random_tensors(specs, seed, std=0.05, dtype=dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    from tiny_inference_server_b200.parts import RMSNormL2
    norm = RMSNormL2(200, 3e-4, prefix="n.")
    w = _random_part_weights(norm, dtype, 0)
    norm.load(w, _ctx(dtype))
    x = torch.randn(7, 200, generator=torch.Generator().manual_seed(0)) * 2
    want = plain_model.plain_rms_norm(x.double(), w["n.scale"].double(), 3e-4)
    got = norm.forward(x.cuda()).cpu().double()
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert float((got - want).abs().max()) < tol


def test_rotary_tables_part():
    from tiny_inference_server_b200.parts import RotaryHalf
    rope = RotaryHalf(48, 25000.0, 300)
    rope.load({}, _ctx(torch.float32))
    cos, sin = plain_model.plain_rope_angles(torch.arange(300), 25000.0, 48)
    assert float((rope.cos.cpu().double() - cos[:, :24]).abs().max()) < 1e-7
    assert float((rope.sin.cpu().double() - sin[:, :24]).abs().max()) < 1e-7


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_part(dtype):
    from tiny_inference_server_b200.parts import SwiGLU
    ffn = SwiGLU(120, 200, prefix="f.")
    w = _random_part_weights(ffn, dtype, 1)
    ffn.load(w, _ctx(dtype))
    x = (torch.randn(9, 120, generator=torch.Generator().manual_seed(1))).to(dtype)
    want = plain_model.plain_swiglu_ffn(x.double(), w["f.swig.linear1.weight"].double(),
                                        w["f.swig.linear2.weight"].double(), w["f.fc.weight"].double())
    got = ffn.forward(x.cuda(), None).cpu().double()
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert float((got - want).abs().max()) < tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [None, 10])
def test_attention_part_in_two_portions(dtype, window):
    """The mixer alone over a cache: 23 positions fed as 14 + 9, against dense attention."""
    from tiny_inference_server_b200.cache import CacheManager
    from tiny_inference_server_b200.engine import build_step, StepEntry
    from tiny_inference_server_b200.parts import GqaAttention, LayerBinding, RotaryHalf
    width, H, KVH, hd, page, T = 72, 6, 2, 32, 4, 23
    rope = RotaryHalf(hd, 10000.0, 64)
    att = GqaAttention(width, H, KVH, hd, rope, window=window, prefix="a.")
    w = _random_part_weights(att, dtype, 2)
    for p in att.walk():
        p.load(w, _ctx(dtype))
    cache = CacheManager([att.kv_spec()], {}, page_size=page, num_pages=16, max_slots=2, max_positions=64,
                         dtype=dtype, device="cuda:0")
    ref = cache.plane_refs[0]
    binding = LayerBinding(kv_plane=cache.groups[ref.group].plane(ref.index), kv_group=ref.group, kv_write=True)
    x = (torch.randn(T, width, generator=torch.Generator().manual_seed(2)) * 0.5).to(dtype)
    fault = torch.zeros(4, dtype=torch.int32, device="cuda")
    slot = cache.admit()
    outs = []
    for a, b in ((0, 14), (14, T)):
        start = cache.extend(slot, b - a)
        cache.sync_tables()
        ctx, _, _ = build_step([StepEntry(slot, [0] * (b - a))], [start], [0], [g.table_dev for g in cache.groups],
                               [page], fault, torch.device("cuda:0"), 10,
                               planners=att.step_planners())
        outs.append(att.forward(x[a:b].cuda(), ctx, binding).cpu())
    got = torch.cat(outs).double()
    xd = x.double()
    q = (xd @ w["a.q_proj.weight"].double()).view(T, H, hd)
    kv = (xd @ w["a.kv_proj.weight"].double()).view(T, 2, KVH, hd)
    cos, sin = plain_model.plain_rope_angles(torch.arange(T), 10000.0, hd)
    o = plain_model.plain_causal_attention(plain_model.plain_apply_rope(q, cos, sin),
                                           plain_model.plain_apply_rope(kv[:, 0], cos, sin), kv[:, 1], window=window)
    want = o.reshape(T, H * hd) @ w["a.linear_proj.weight"].double()
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert float((got - want).abs().max()) < tol
    assert int(fault[0]) == 0


# ----------------------------------------------------------------------------------------
# a toy mixer with state of its own
# ----------------------------------------------------------------------------------------

def test_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path):
    """A decaying running sum, s <- 0.5 s + x W, y = s: no keys and values, one state row per
    request.  It is defined here, registered, named by the configuration for layer 1, given
    random weights by the engine's random-weights mode, and stepped whole, token by token
    and in portions; the logits agree with a plain computation."""
    from tiny_inference_server_b200 import register_part
    from tiny_inference_server_b200.config import EngineConfig
    from tiny_inference_server_b200.engine import ModelRunner, StepEntry
    from tiny_inference_server_b200.parts import Mixer, StateSpec, WeightSpec

    class ToyDecay(Mixer):
        def __init__(self, width, prefix=""):
            super().__init__(prefix)
            self.width = width
            self.w = None

        @classmethod
        def from_config(cls, cfg, prefix, layer_index, lag, position=None):
            return cls(cfg.hidden_size, prefix=prefix)

        def state_spec(self):
            return StateSpec((self.width,), torch.float32)

        def weight_specs(self):
            return {"toy.weight": WeightSpec((self.width, self.width))}

        def load(self, tensors, ctx):
            self.w = tensors[self.prefix + "toy.weight"].to(device=ctx.device, dtype=torch.float32)

        def forward(self, x, step, binding):
            u = x.float() @ self.w
            out = torch.empty_like(u)
            for seg in step.segments:                  # rows of a request are contiguous and in order
                s = binding.state[seg.slot]
                for r in range(seg.row0, seg.row0 + seg.rows):
                    s = 0.5 * s + u[r]
                    out[r] = s
                binding.state[seg.slot] = s
            return out.to(x.dtype)

    register_part("mixer", "toy_decay", ToyDecay)
    cfg = dict(tiny_configs.TINY_A, mixer_types=["gqa", "toy_decay"], num_mtp_heads=0)
    folder = tiny_configs.make_model_folder(cfg, 4, str(tmp_path / "toy"))
    c, W = plain_model.read_config(folder), plain_model.read_weights(folder)
    toks = tiny_configs.random_prompts(cfg["vocab_size"], [21], seed=12)[0]

    # plain computation: layer 0 is the ordinary block, layer 1 has the toy mixer
    ids = torch.tensor(toks)
    x = W["embedding.weight"][ids]
    x, _ = plain_model.plain_block(x, W, "transformer_block_list.0.", c, torch.arange(len(toks)), None)
    pre = "transformer_block_list.1."
    a = plain_model.plain_rms_norm(x, W[pre + "att.rms_norm_att.scale"], c["rms_norm_eps"])
    u = a @ W[pre + "att.toy.weight"]
    s = torch.zeros(c["hidden_size"], dtype=torch.float64)
    ys = []
    for r in range(len(toks)):
        s = 0.5 * s + u[r]
        ys.append(s)
    x = x + torch.stack(ys)
    f = plain_model.plain_rms_norm(x, W[pre + "rms_norm_ffn.scale"], c["rms_norm_eps"])
    x = x + plain_model.plain_swiglu_ffn(f, W[pre + "ffn.swig.linear1.weight"], W[pre + "ffn.swig.linear2.weight"],
                                         W[pre + "ffn.fc.weight"])
    want = plain_model.plain_logits(c, W, plain_model.plain_rms_norm(x, W["rms_out.scale"], c["rms_norm_eps"]))

    for cuts in ([21], [1] * 21, [5, 2, 9, 3, 2]):
        r = ModelRunner.from_folder(folder, EngineConfig(dtype="float32", page_size=16, num_pages=8))
        assert "entry1" in r.cache.states and r.cache.plane_refs[1] is None
        slot = r.add_request()
        other = r.add_request()                       # a second request beside it must not disturb its state
        got, p = [], 0
        for n in cuts:
            out = r.step([StepEntry(other, [1]), StepEntry(slot, toks[p:p + n], list(range(n)))])
            got.append(out.main.cpu())
            p += n
        got = torch.cat(got).double()
        assert float((got - want).abs().max()) < 2e-4, cuts
        r.release(slot)
        r.release(other)
        assert r.cache.drained()
