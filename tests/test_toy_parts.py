"""Parts and an architecture defined here, in a test, are registered, built from ``config.json``,
given random weights by the engine's random-weights mode, loaded by tensor name and stepped —
whole, token by token and in portions — with no change to a file of the package:

* a position encoding of another kind ("none": no rotation, the cache write only);
* a norm of another form (rsqrt(mean of squares + eps)), which the decode products fold into themselves as they do
  the architecture's own;
* a feed-forward with routing (two experts, the better one per token);
* a mixer whose cached keys and values have different widths (a key of 8, a value of 24 elements);
* a whole architecture with tensor names of its own (``register_architecture``).

None of them is a model of anyone's; they show what the interfaces allow.  Each runs on the CPU
(with the plain references in place of the kernels) and, marked ``gpu``, on the device."""
import dataclasses
import json
import math
import os

import pytest
import torch

import plain_model
import tiny_configs

DEVICES = ["cpu", pytest.param("cuda:0", marks=pytest.mark.gpu)]
CUTS = ([19], [1] * 19, [5, 2, 9, 3])


def _runner(folder, device, request, **kw):
    from tiny_inference_server_b200.config import EngineConfig
    from tiny_inference_server_b200.engine import ModelRunner
    if device == "cpu":
        request.getfixturevalue("ref_ops")
    base = dict(dtype="float32", page_size=8, num_pages=16, device=device, cuda_graphs=device != "cpu")
    base.update(kw)
    return ModelRunner.from_folder(folder, EngineConfig(**base))


def _step_through(runner, toks, cuts):
    """Feed ``toks`` in portions of ``cuts`` beside a second request; the logits of every position."""
    from tiny_inference_server_b200.engine import StepEntry
    slot, other = runner.add_request(), runner.add_request()
    got, p = [], 0
    for n in cuts:
        out = runner.step([StepEntry(other, [1]), StepEntry(slot, toks[p:p + n], list(range(n)))])
        got.append(out.main.float().cpu())
        p += n
    runner.check_fault()
    runner.release(slot)
    runner.release(other)
    assert runner.cache.drained()
    return torch.cat(got).double()


# ---------------------------------------------------------------------------------------------------
# a position encoding of another kind
# ---------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("device", DEVICES)
def test_toy_position_encoding_without_rotation(device, tmp_path, request, monkeypatch):
    from tiny_inference_server_b200 import register_part
    from tiny_inference_server_b200.kernels import ops
    from tiny_inference_server_b200.parts import PositionEncoding

    class NoPosition(PositionEncoding):
        """Queries and keys as they are: only the cache write is left of ``encode_and_store``."""

        def __init__(self, head_dim, max_positions):
            super().__init__("")
            self.head_dim, self.max_positions = head_dim, max_positions
            self.one = self.zero = None

        @classmethod
        def from_config(cls, cfg):
            return cls(cfg.head_dim, cfg.max_context)

        def load(self, tensors, ctx):
            self.one = torch.ones(self.max_positions, self.head_dim // 2, dtype=torch.float32, device=ctx.device)
            self.zero = torch.zeros_like(self.one)

        def encode_and_store(self, qkv, step, *, num_heads, kv_heads, head_dim, plane, block_table, page_size):
            # a rotation by the angle zero: the engine's kernel writes the rows into their pages
            ops.rope_kv_write(qkv, step.positions, step.row_slot, self.one, self.zero, plane, block_table, num_heads,
                              kv_heads, head_dim, page_size, step.fault, write_kv=plane is not None)

    register_part("position", "toy_none", NoPosition)
    cfg = dict(tiny_configs.TINY_B, position_type="toy_none")
    folder = tiny_configs.make_model_folder(cfg, 3, str(tmp_path / "m"))
    c, W = plain_model.read_config(folder), plain_model.read_weights(folder)
    toks = tiny_configs.random_prompts(cfg["vocab_size"], [19], seed=5)[0]
    with_rope = plain_model.plain_forward(c, W, toks, mtp=False)["main"]
    monkeypatch.setattr(plain_model, "plain_rope_angles",
                        lambda positions, theta, hd: (torch.ones(len(positions), hd, dtype=torch.float64),
                                                      torch.zeros(len(positions), hd, dtype=torch.float64)))
    want = plain_model.plain_forward(c, W, toks, mtp=False)["main"]
    assert float((want - with_rope).abs().max()) > 1e-3          # the rotation matters for this model
    for cuts in CUTS:
        got = _step_through(_runner(folder, device, request), toks, cuts)
        assert float((got - want).abs().max()) < 2e-4, cuts


# ---------------------------------------------------------------------------------------------------
# a norm of another form
# ---------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("device", DEVICES)
def test_toy_norm_of_another_form(device, tmp_path, request, monkeypatch):
    """y = x * rsqrt(mean(x^2) + eps) * scale, with a large eps so that its place matters.  Whole, the norm runs as
    the part's own operations; token by token in bfloat16 the last product of every mixer and feed-forward adds to
    the stream itself and the next product applies this norm's factor (the sink the norm hands out names it)."""
    from tiny_inference_server_b200 import register_part
    from tiny_inference_server_b200.kernels import ops
    from tiny_inference_server_b200.parts import Norm, WeightSpec

    class MeanSquareNorm(Norm):
        def __init__(self, width, eps, prefix=""):
            super().__init__(prefix)
            self.width, self.eps = width, float(eps)
            self.scale, self.out_dtype = None, torch.float32

        @classmethod
        def from_config(cls, cfg, prefix):
            return cls(cfg.hidden_size, cfg.rms_norm_eps, prefix=prefix)

        def weight_specs(self):
            return {"scale": WeightSpec((self.width,), init="ones_normal")}

        def load(self, tensors, ctx):
            self.scale = tensors[self.prefix + "scale"].to(device=ctx.device, dtype=torch.float32).contiguous()
            self.out_dtype = ctx.dtype

        def add_norm(self, residual, delta):
            if delta is not None:
                residual += delta.float()
            return (residual * torch.rsqrt(residual.pow(2).mean(-1, keepdim=True) + self.eps) * self.scale).to(self.out_dtype)

        def forward(self, residual):
            return self.add_norm(residual, None)

        def sink(self, values):
            return ops.ResidualSink(values, self.scale, self.eps, norm=self, kind="mean_eps")

    register_part("norm", "toy_mean_square", MeanSquareNorm)
    cfg = dict(tiny_configs.TINY_A, norm_type="toy_mean_square", rms_norm_eps=0.5, num_mtp_heads=0)
    folder = tiny_configs.make_model_folder(cfg, 8, str(tmp_path / "m"))
    c, W = plain_model.read_config(folder), plain_model.read_weights(folder)
    toks = tiny_configs.random_prompts(cfg["vocab_size"], [19], seed=9)[0]
    own_form = plain_model.plain_forward(c, W, toks, mtp=False)["main"]
    monkeypatch.setattr(plain_model, "plain_rms_norm",
                        lambda x, scale, eps: x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * scale)
    want = plain_model.plain_forward(c, W, toks, mtp=False)["main"]
    assert float((want - own_form).abs().max()) > 0.05           # the form of the norm matters for this model
    for cuts in CUTS:
        got = _step_through(_runner(folder, device, request), toks, cuts)
        assert float((got - want).abs().max()) < 2e-4, cuts
    # bfloat16, token by token: the norms are folded into the products (a sink per mixer and feed-forward but the last)
    sinks = []
    made = ops.ResidualSink.__init__

    def counted(self, *a, **k):
        sinks.append(k.get("kind"))
        made(self, *a, **k)
    monkeypatch.setattr(ops.ResidualSink, "__init__", counted)
    got = _step_through(_runner(folder, device, request, dtype="bfloat16"), toks, [1] * 19)
    # (on the device the step is captured into a graph once and replayed: the sinks are made at the capture)
    steps_in_python = 19 if device == "cpu" else 1
    assert len(sinks) >= steps_in_python * (2 * cfg["num_layers"] - 1) and set(sinks) == {"mean_eps"}
    assert float((got - want).abs().max()) < 3e-2
    monkeypatch.setattr(ops, "FUSED_NORM", False)
    unfused = _step_through(_runner(folder, device, request, dtype="bfloat16"), toks, [1] * 19)
    assert float((unfused - want).abs().max()) < 3e-2 and float((unfused - got).abs().max()) < 3e-2


# ---------------------------------------------------------------------------------------------------
# a feed-forward with routing
# ---------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("device", DEVICES)
def test_toy_routed_feed_forward(device, tmp_path, request):
    from tiny_inference_server_b200 import register_part
    from tiny_inference_server_b200.parts import FeedForward, WeightSpec

    class ToyExperts(FeedForward):
        """y = p_e * relu(x A_e) B_e for the expert e with the larger router logit (router in float32)."""

        def __init__(self, width, hidden, prefix=""):
            super().__init__(prefix)
            self.width, self.hidden = width, hidden
            self.router = self.a = self.b = None

        @classmethod
        def from_config(cls, cfg, prefix, layer_index):
            return cls(cfg.hidden_size, cfg.ffn_hidden // 2, prefix=prefix)

        def weight_specs(self):
            return {"router.weight": WeightSpec((self.width, 2)), "experts.a": WeightSpec((2, self.width, self.hidden)),
                    "experts.b": WeightSpec((2, self.hidden, self.width))}

        def load(self, tensors, ctx):
            def get(n):
                return tensors[self.prefix + n].to(device=ctx.device, dtype=torch.float32)
            self.router, self.a, self.b = get("router.weight"), get("experts.a"), get("experts.b")

        def forward(self, x, step=None):
            x32 = x.float()
            p = torch.softmax(x32 @ self.router, dim=-1)
            e = p.argmax(dim=-1)
            h = torch.relu(torch.einsum("nd,ndh->nh", x32, self.a[e]))
            return (p.gather(1, e[:, None]) * torch.einsum("nh,nhd->nd", h, self.b[e])).to(x.dtype)

    register_part("ffn", "toy_experts", ToyExperts)
    cfg = dict(tiny_configs.TINY_A, ffn_types=["toy_experts", "swiglu"], num_mtp_heads=0)
    folder = tiny_configs.make_model_folder(cfg, 6, str(tmp_path / "m"), std=0.2)
    c, W = plain_model.read_config(folder), plain_model.read_weights(folder)
    toks = tiny_configs.random_prompts(cfg["vocab_size"], [19], seed=7)[0]

    # plain computation: block 0 with the routed feed-forward, block 1 as it is
    T = len(toks)
    pos = torch.arange(T)
    x = W["embedding.weight"][torch.tensor(toks)]
    pre = "transformer_block_list.0."
    a = plain_model.plain_rms_norm(x, W[pre + "att.rms_norm_att.scale"], c["rms_norm_eps"])
    q = (a @ W[pre + "att.q_proj.weight"]).view(T, c["num_heads"], c["head_dim"])
    cos, sin = plain_model.plain_rope_angles(pos, c["rope_theta"], c["head_dim"])
    k, v = plain_model._kv_project(a, W, pre, c)
    o = plain_model.plain_causal_attention(plain_model.plain_apply_rope(q, cos, sin),
                                           plain_model.plain_apply_rope(k, cos, sin), v)
    x = x + o.reshape(T, -1) @ W[pre + "att.linear_proj.weight"]
    f = plain_model.plain_rms_norm(x, W[pre + "rms_norm_ffn.scale"], c["rms_norm_eps"])
    p = torch.softmax(f @ W[pre + "ffn.router.weight"], dim=-1)
    e = p.argmax(dim=-1)
    assert 0 < int(e.sum()) < T, "both experts must be chosen by some token"
    h = torch.relu(torch.einsum("nd,ndh->nh", f, W[pre + "ffn.experts.a"][e]))
    x = x + p.gather(1, e[:, None]) * torch.einsum("nh,nhd->nd", h, W[pre + "ffn.experts.b"][e])
    x, _ = plain_model.plain_block(x, W, "transformer_block_list.1.", c, pos, None)
    want = plain_model.plain_logits(c, W, plain_model.plain_rms_norm(x, W["rms_out.scale"], c["rms_norm_eps"]))
    for cuts in CUTS:
        got = _step_through(_runner(folder, device, request, page_size=16), toks, cuts)
        assert float((got - want).abs().max()) < 5e-4 * max(1.0, float(want.abs().max())), cuts


# ---------------------------------------------------------------------------------------------------
# a mixer whose keys and values differ in width
# ---------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("device", DEVICES)
def test_toy_mixer_with_keys_and_values_of_different_widths(device, tmp_path, request):
    from tiny_inference_server_b200 import register_part
    from tiny_inference_server_b200.parts import KVSpec, Mixer, WeightSpec

    KD, VD = 8, 24

    class NarrowKeys(Mixer):
        """One head: q, k of 8 elements, v of 24; causal softmax attention over the paged cache, written
        and read here with plain indexing through the block table (pages [kv head, position, width])."""

        def __init__(self, width, prefix=""):
            super().__init__(prefix)
            self.width = width
            self.wq = self.wk = self.wv = self.wo = None

        @classmethod
        def from_config(cls, cfg, prefix, layer_index, lag, position=None):
            return cls(cfg.hidden_size, prefix=prefix)

        def kv_spec(self):
            return KVSpec(kv_heads=1, head_dim=KD, k_dim=KD, v_dim=VD)

        def weight_specs(self):
            return {"wq": WeightSpec((self.width, KD)), "wk": WeightSpec((self.width, KD)),
                    "wv": WeightSpec((self.width, VD)), "wo": WeightSpec((VD, self.width))}

        def load(self, tensors, ctx):
            for n in ("wq", "wk", "wv", "wo"):
                setattr(self, n, tensors[self.prefix + n].to(device=ctx.device, dtype=torch.float32))

        def forward(self, x, step, binding):
            assert binding.kv_plane is None and binding.k_pages.shape[-1] == KD and binding.v_pages.shape[-1] == VD
            x32 = x.float()
            q, k, v = x32 @ self.wq, x32 @ self.wk, x32 @ self.wv
            table, page = step.block_tables[binding.kv_group], step.page_sizes[binding.kv_group]
            out = torch.zeros(x.shape[0], VD, dtype=torch.float32, device=x.device)
            for seg in step.segments:
                pages = table[seg.slot].long()
                for i in range(seg.rows):
                    r, p = seg.row0 + i, seg.pos0 + i
                    binding.k_pages[pages[p // page], 0, p % page] = k[r].to(binding.k_pages.dtype)
                    binding.v_pages[pages[p // page], 0, p % page] = v[r].to(binding.v_pages.dtype)
                    idx = torch.arange(p + 1, device=x.device)
                    ks = binding.k_pages[pages[idx // page], 0, idx % page].float()
                    vs = binding.v_pages[pages[idx // page], 0, idx % page].float()
                    out[r] = torch.softmax(ks @ q[r] / math.sqrt(KD), dim=0) @ vs
            return (out @ self.wo).to(x.dtype)

    register_part("mixer", "toy_narrow_keys", NarrowKeys)
    cfg = dict(tiny_configs.TINY_A, mixer_types=["toy_narrow_keys", "gqa"], num_mtp_heads=0)
    folder = tiny_configs.make_model_folder(cfg, 8, str(tmp_path / "m"), std=0.2)
    c, W = plain_model.read_config(folder), plain_model.read_weights(folder)
    toks = tiny_configs.random_prompts(cfg["vocab_size"], [19], seed=9)[0]
    T = len(toks)
    x = W["embedding.weight"][torch.tensor(toks)]
    pre = "transformer_block_list.0."
    a = plain_model.plain_rms_norm(x, W[pre + "att.rms_norm_att.scale"], c["rms_norm_eps"])
    q, k, v = a @ W[pre + "att.wq"], a @ W[pre + "att.wk"], a @ W[pre + "att.wv"]
    s = (q @ k.T / math.sqrt(KD)).masked_fill(~torch.tril(torch.ones(T, T, dtype=torch.bool)), float("-inf"))
    x = x + (torch.softmax(s, -1) @ v) @ W[pre + "att.wo"]
    f = plain_model.plain_rms_norm(x, W[pre + "rms_norm_ffn.scale"], c["rms_norm_eps"])
    x = x + plain_model.plain_swiglu_ffn(f, W[pre + "ffn.swig.linear1.weight"], W[pre + "ffn.swig.linear2.weight"],
                                         W[pre + "ffn.fc.weight"])
    x, _ = plain_model.plain_block(x, W, "transformer_block_list.1.", c, torch.arange(T), None)
    want = plain_model.plain_logits(c, W, plain_model.plain_rms_norm(x, W["rms_out.scale"], c["rms_norm_eps"]))
    for cuts in CUTS:
        runner = _runner(folder, device, request, page_size=4, num_pages=24)
        # two groups: the toy's pages of 1 x 4 x (8 + 24) elements, the ordinary layer's pages
        widths = sorted((g.head_dim, g.v_dim) for g in runner.cache.groups)
        assert widths == [(KD, VD), (c["head_dim"], c["head_dim"])]
        got = _step_through(runner, toks, cuts)
        assert float((got - want).abs().max()) < 5e-4 * max(1.0, float(want.abs().max())), cuts


# ---------------------------------------------------------------------------------------------------
# a whole architecture
# ---------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("device", DEVICES)
def test_toy_architecture_is_registered_from_outside(device, tmp_path, request):
    from tiny_inference_server_b200 import ConfigError, register_architecture
    from tiny_inference_server_b200.models.base import Model, ScheduleEntry, StepOutput
    from tiny_inference_server_b200.parts import (Block, Embedding, GqaAttention, LMHead, ResidualStream, RMSNormL2,
                                                  RotaryHalf, SwiGLU)
    from tiny_inference_server_b200.registry import config_from_folder
    from tiny_inference_server_b200.weights import write_random_model

    @dataclasses.dataclass
    class ToyConfig:
        architecture = "toy_two_tower"
        vocab: int
        width: int
        heads: int
        depth: int
        inner: int
        eps: float = 1e-5
        base: float = 10000.0
        context: int = 64
        torch_dtype: str = "bfloat16"

        @classmethod
        def from_dict(cls, raw):
            raw = {k: v for k, v in raw.items() if k != "architecture"}
            unknown = sorted(set(raw) - {f.name for f in dataclasses.fields(cls)})
            if unknown:
                raise ConfigError(f"toy_two_tower: unknown keys {unknown}")
            return cls(**raw)

        def to_dict(self):
            return dict(dataclasses.asdict(self), architecture=self.architecture)

    class ToyModel(Model):
        """Embedding, ``depth`` blocks of multi-head attention and SwiGLU, norm, an output matrix of its
        own; the last block's attention reads the cache of the first.  Tensor names of its own."""

        def __init__(self, cfg):
            super().__init__()
            self.config, self.vocab_size, self.max_positions = cfg, cfg.vocab, cfg.context
            hd = cfg.width // cfg.heads
            self.rope = RotaryHalf(hd, cfg.base, cfg.context)
            self.wte = Embedding(cfg.vocab, cfg.width, weight_name="wte")
            self.blocks = [
                Block(RMSNormL2(cfg.width, cfg.eps, prefix=f"h.{l}.ln1.", weight_name="g"),
                      GqaAttention(cfg.width, cfg.heads, cfg.heads, hd, self.rope, prefix=f"h.{l}.attn.",
                                   names={"q": "wq", "kv": "wkv", "o": "wo"}),
                      RMSNormL2(cfg.width, cfg.eps, prefix=f"h.{l}.ln2.", weight_name="g"),
                      SwiGLU(cfg.width, cfg.inner, prefix=f"h.{l}.mlp.", names={"gate": "w1", "up": "w2", "down": "w3"}),
                      prefix=f"h.{l}.")
                for l in range(cfg.depth)]
            self.ln_f = RMSNormL2(cfg.width, cfg.eps, prefix="ln_f.", weight_name="g")
            self.head = LMHead(cfg.vocab, cfg.width, None, weight_name="head")
            self.entries = [ScheduleEntry(b) for b in self.blocks]
            self.entries[-1].source = 0

        def top_parts(self):
            return [self.wte, self.rope, *self.blocks, self.ln_f, self.head]

        def forward(self, step, want_rows, aux=False):
            stream = ResidualStream(self.wte.forward(step.tokens))
            for e in self.entries:
                e.block.forward(stream, step, e.binding)
            return StepOutput(main=self.head.forward(stream.normed(self.ln_f).index_select(0, want_rows)))

    register_architecture("toy_two_tower", ToyConfig, ToyModel)
    cfg = ToyConfig(vocab=150, width=48, heads=3, depth=3, inner=72, eps=2e-6, base=5000.0)
    folder = write_random_model(str(tmp_path / "toy"), cfg, seed=10, std=0.1)
    assert json.load(open(os.path.join(folder, "config.json")))["architecture"] == "toy_two_tower"
    assert isinstance(config_from_folder(folder), ToyConfig)
    with pytest.raises(ConfigError, match="unknown keys"):
        from tiny_inference_server_b200 import config_from_dict
        config_from_dict(dict(cfg.to_dict(), colour=1))

    W = plain_model.read_weights(folder)
    toks = tiny_configs.random_prompts(cfg.vocab, [19], seed=11)[0]
    T, hd = len(toks), cfg.width // cfg.heads
    pos = torch.arange(T)
    cos, sin = plain_model.plain_rope_angles(pos, cfg.base, hd)
    x = W["wte"][torch.tensor(toks)]
    kept = None
    for l in range(cfg.depth):
        a = plain_model.plain_rms_norm(x, W[f"h.{l}.ln1.g"], cfg.eps)
        q = plain_model.plain_apply_rope((a @ W[f"h.{l}.attn.wq"]).view(T, cfg.heads, hd), cos, sin)
        if l == cfg.depth - 1:
            k, v = kept
        else:
            kv = (a @ W[f"h.{l}.attn.wkv"]).view(T, 2, cfg.heads, hd)
            k, v = plain_model.plain_apply_rope(kv[:, 0], cos, sin), kv[:, 1]
            if l == 0:
                kept = (k, v)
        x = x + plain_model.plain_causal_attention(q, k, v).reshape(T, -1) @ W[f"h.{l}.attn.wo"]
        f = plain_model.plain_rms_norm(x, W[f"h.{l}.ln2.g"], cfg.eps)
        x = x + plain_model.plain_swiglu_ffn(f, W[f"h.{l}.mlp.w1"], W[f"h.{l}.mlp.w2"], W[f"h.{l}.mlp.w3"])
    want = plain_model.plain_rms_norm(x, W["ln_f.g"], cfg.eps) @ W["head"].T
    for cuts in CUTS:
        runner = _runner(folder, device, request)
        assert len(runner.cache.groups) == 1 and runner.cache.groups[0].num_planes == cfg.depth - 1
        got = _step_through(runner, toks, cuts)
        assert float((got - want).abs().max()) < 5e-4 * max(1.0, float(want.abs().max())), cuts
