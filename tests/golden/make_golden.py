"""Makes tests/golden/reference_tiny.npz: logits of the upstream project's own model code
on a tiny random model, to anchor tests/plain_model.py once.

Run on the CPU:  python tests/golden/make_golden.py /path/to/upstream/checkout

The upstream modules (``main_models_new.Transformer`` with its ``paged_gqa``,
``Transformer_block``, ``mtp_head``, ``rms_norm``, RoPE tables, and ``block_table``) are
imported unchanged.  Its three Triton entry points cannot run without a GPU, so three
names of ``main_models_new`` are rebound to plain torch stand-ins (a page write, dense
attention over a page table, dense causal attention over packed prompts); everything
else — norm form, weight layouts, the K/V split of ``kv_proj``, rotary encoding, the MTP
wiring, ``prefill_rows`` / ``mtp_prefill_rows`` / ``trunk_rows`` — is upstream's code.

The attention formula itself (scale 1/sqrt(head size), the causal rule, query head h reading
kv head h // group) is pinned by a fourth array, ``dense_main``: the logits of upstream's own
pure-torch dense oracle, ``dense_forward`` of its ``test_server.py`` (lines 23-45:
``F.scaled_dot_product_attention(is_causal=True)`` after ``repeat_interleave``), with no
stand-in on its path.  That file runs GPU tests when imported, so only the text of that one
function is taken out of it and executed with the globals it reads (``NH, HD, KVH, GROUP, D``,
``rotate_half``) set from this configuration.
The weights are this repository's random weights (seeded), copied into upstream's
parameters by name; upstream's eps buffers are set to the configuration's eps.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.normpath(os.path.join(HERE, os.pardir)))
sys.path.insert(0, os.path.normpath(os.path.join(HERE, os.pardir, os.pardir)))

CFG = dict(architecture="gqa_mtp_transformer", vocab_size=256, hidden_size=64, num_layers=2, num_heads=4,
           num_kv_heads=2, ffn_hidden=192, rms_norm_eps=1e-5, rope_theta=10000.0, max_context=128,
           tie_word_embeddings=True, num_mtp_heads=2, torch_dtype="float32")
SEED = 1234
TOKENS = [5, 200, 17, 3, 99, 250, 0, 42, 42, 7, 131, 64, 8]
NEXT = 77          # one decode row after the prompt, through upstream's paged path
TPB = 16


def upstream_dense_forward(upstream: str, M, c):
    """Upstream's ``dense_forward`` (test_server.py:23-45), compiled from its own source text."""
    import torch.nn.functional as F
    src = open(os.path.join(upstream, "test_server.py")).read()
    a = src.index("@torch.no_grad()\ndef dense_forward")
    b = src.index("\ndef ", a + 30)
    hd = c["hidden_size"] // c["num_heads"]
    env = dict(torch=torch, F=F, rotate_half=M.rotate_half, NH=c["num_heads"], HD=hd, KVH=c["num_kv_heads"],
               GROUP=c["num_heads"] // c["num_kv_heads"], D=c["hidden_size"])
    exec(compile(src[a:b], os.path.join(upstream, "test_server.py"), "exec"), env)
    return env["dense_forward"]


def main(upstream: str):
    sys.path.insert(0, upstream)
    sys.dont_write_bytecode = True
    import main_models_new as M
    import block_table as BT
    import tempfile
    from safetensors.torch import load_file
    import tiny_configs

    class _WriteKV:
        def __getitem__(self, grid):
            def run(pool_layer, write_ptrs, k, v, kv_stride, head_stride, HEAD_DIM):
                flat = pool_layer.reshape(-1)
                assert flat.data_ptr() == pool_layer.data_ptr()
                n, kvh, hd = k.shape
                for b in range(n):
                    for h in range(kvh):
                        o = int(write_ptrs[b]) + h * head_stride
                        flat[o:o + hd] = k[b, h]
                        flat[o + kv_stride:o + kv_stride + hd] = v[b, h]
            return run

    def paged_standin(q, page_table, pool, kv_lens, group_size, page_starts, max_seq_len, layer=0):
        n, H, hd = q.shape
        out = torch.empty_like(q)
        tpb = pool.tokens_per_block
        for b in range(n):
            L = int(kv_lens[b])
            npg = (L + tpb - 1) // tpb
            st = int(page_starts[b])
            pages = page_table[st:st + npg].long()
            k = pool.block[layer, :, 0, pages].reshape(pool.num_heads, -1, hd)[:, :L]
            v = pool.block[layer, :, 1, pages].reshape(pool.num_heads, -1, hd)[:, :L]
            k = k.repeat_interleave(group_size, 0)
            v = v.repeat_interleave(group_size, 0)
            s = torch.einsum("hd,hld->hl", q[b], k) / hd ** 0.5
            out[b] = torch.einsum("hl,hld->hd", torch.softmax(s, -1), v)
        return out

    def intradoc_standin(q, k, v, cuseq, max_len, group_size):
        out = torch.empty_like(q)
        cs = cuseq.tolist()
        hd = q.shape[-1]
        for a, b in zip(cs, cs[1:]):
            if b == a:
                continue
            qq = q[a:b].transpose(0, 1)
            kk = k[a:b].transpose(0, 1).repeat_interleave(group_size, 0)
            vv = v[a:b].transpose(0, 1).repeat_interleave(group_size, 0)
            s = qq @ kk.transpose(1, 2) / hd ** 0.5
            s = s.masked_fill(~torch.tril(torch.ones(b - a, b - a, dtype=torch.bool)), float("-inf"))
            out[a:b] = (torch.softmax(s, -1) @ vv).transpose(0, 1)
        return out, None

    M.write_kv_cache_decode = _WriteKV()
    M.paged_flash_decode = paged_standin
    M.triton_intradoc_attention = intradoc_standin

    c = CFG
    group = c["num_heads"] // c["num_kv_heads"]
    hd = c["hidden_size"] // c["num_heads"]
    with tempfile.TemporaryDirectory() as tmp:
        folder = tiny_configs.make_model_folder(c, SEED, tmp)
        W = load_file(os.path.join(folder, "model.safetensors"))
    m = M.Transformer(c["vocab_size"], c["max_context"], c["rope_theta"], c["hidden_size"], c["num_heads"],
                      c["num_layers"], c["ffn_hidden"], group, mtp_heads=c["num_mtp_heads"]).eval()
    names = dict(m.named_parameters())
    assert set(names) == set(W), (sorted(set(names) ^ set(W)))
    with torch.no_grad():
        for n_, p in names.items():
            assert tuple(p.shape) == tuple(W[n_].shape), n_
            p.copy_(W[n_].float())
        for mod in m.modules():
            if isinstance(mod, M.rms_norm):
                mod.eps.fill_(c["rms_norm_eps"])

    planes = c["num_layers"] + c["num_mtp_heads"]
    page_elems = TPB * 2 * 2 * c["num_kv_heads"] * planes * hd
    pool = BT.block_table(planes, c["num_kv_heads"], hd, 16 * page_elems, TPB, "cpu")
    pool.block = pool.block.float()
    user = BT.User(pool)
    T = len(TOKENS)
    toks = torch.tensor(TOKENS)
    pos = torch.arange(T)
    with torch.no_grad():
        wp = torch.tensor([user.slot(p) for p in range(T)])
        h = m.prefill_rows(toks, pool, pos, wp, torch.tensor([0, T], dtype=torch.int32), T)
        main = m.logits(h)
        mtp = []
        prev = h
        for i in range(c["num_mtp_heads"]):
            n = T - 1 - i
            prev = m.mtp_prefill_rows(i, prev[:n], toks[1 + i:1 + i + n], pool, pos[:n], wp[:n],
                                      torch.tensor([0, n], dtype=torch.int32), n)
            mtp.append(m.logits(prev))
        # one decode row over the pages the prefill wrote (upstream trunk_rows)
        w1 = torch.tensor([user.slot(T)])
        hd1 = m.trunk_rows(torch.tensor([NEXT]), pool, torch.tensor(user.block_ids, dtype=torch.int32),
                           torch.tensor([0], dtype=torch.int32), torch.tensor([T]),
                           torch.tensor([T + 1], dtype=torch.int32), w1, T + 1)
        decode = m.logits(hd1)
        # upstream's dense oracle, no stand-in on its path; it must agree with upstream's own
        # prefill path (which ran on the stand-ins) before it is written
        dense = upstream_dense_forward(upstream, M, c)(m, toks)
        assert float((dense - main).abs().max()) < 5e-6, float((dense - main).abs().max())
    out = os.path.join(HERE, "reference_tiny.npz")
    np.savez_compressed(out, main=main.numpy(), mtp0=mtp[0].numpy(), mtp1=mtp[1].numpy(), decode=decode.numpy(),
                        dense_main=dense.numpy(), tokens=np.array(TOKENS), next=np.array([NEXT]), seed=np.array([SEED]))
    print("wrote", out, {k: v.shape for k, v in dict(main=main, mtp0=mtp[0], mtp1=mtp[1], decode=decode, dense_main=dense).items()})


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py UPSTREAM_CHECKOUT")
    main(sys.argv[1])
