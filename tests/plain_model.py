"""Plain, slow implementation of the GQA decoder with multi-token-prediction heads.

Whole sequences, no cache, one function per part, no code shared with the engine
package: this file reads ``config.json`` and ``model.safetensors`` on its own and
computes everything with ordinary tensor arithmetic in one dtype (float64 by
default, so that its own rounding is negligible beside the engine's).

Every function is written from the formulas of the upstream project's model code
and cites the place (path within that project, ``file:line``).  The one-off
comparison of this file with the upstream modules on a tiny random model lives in
``tests/golden/`` (script and its committed outputs).

Options that the upstream model does not have (an untied output matrix, a key
window, a layer order that repeats layers or lets a layer read another layer's
keys and values) are the engine's own; their formulas are stated where they are
computed.
"""
from __future__ import annotations

import json
import math
import os

import torch

# --------------------------------------------------------------------------------------
# configuration and weights (read independently of the engine package)
# --------------------------------------------------------------------------------------

_UPSTREAM_NAMES = {
    # Config/config.py:11-23 of the upstream project
    "D_MODEL": "hidden_size", "VOCAB_SIZE": "vocab_size", "MAX_CONTEXT": "max_context",
    "MAX_FREQ": "rope_theta", "N_HEAD": "num_heads", "NUM_LAYERS": "num_layers",
    "FFN_HIDDEN_DIM": "ffn_hidden", "MTP_HEADS": "num_mtp_heads",
}


def read_config(folder: str) -> dict:
    with open(os.path.join(folder, "config.json")) as f:
        raw = json.load(f)
    c = {}
    for k, v in raw.items():
        c[_UPSTREAM_NAMES.get(k, k)] = v
    if "NUM_GROUPS" in c:  # Config/config.py:22 — really the number of query heads per kv head
        c["num_kv_heads"] = c["num_heads"] // c.pop("NUM_GROUPS")
    c.setdefault("head_dim", c["hidden_size"] // c["num_heads"])  # main_models_new.py:91
    c.setdefault("rms_norm_eps", 2e-8)  # main_models_new.py:36
    c.setdefault("rope_theta", 10000.0)
    c.setdefault("tie_word_embeddings", True)
    c.setdefault("num_mtp_heads", 0)
    c.setdefault("sliding_window", None)
    c.setdefault("full_attention_layers", None)
    c.setdefault("layer_order", None)
    c.setdefault("cache_source", None)
    return c


def read_weights(folder: str, dtype=torch.float64) -> dict:
    from safetensors.torch import load_file
    return {k: v.to(dtype) for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}


# --------------------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------------------

def plain_rms_norm(x, scale, eps):
    """main_models_new.py:38-42 — x * sqrt(d) / (||x||_2 + eps) * scale.

    eps is added to the L2 norm itself, not under a square root of a mean.
    """
    d = x.shape[-1]
    norm = torch.sqrt((x * x).sum(-1, keepdim=True))
    return x * math.sqrt(d) / (norm + eps) * scale


def plain_rope_angles(positions, theta, head_dim):
    """main_models_new.py:63-69 — angle[pos, i] = pos * theta^(-2i/hd), i in [0, hd/2);
    the cos and sin tables repeat the half twice along the last axis."""
    i = torch.arange(0, head_dim // 2, dtype=torch.float64)
    inv = 1.0 / torch.pow(torch.tensor(float(theta), dtype=torch.float64), 2 * i / head_dim)
    ang = torch.outer(positions.to(torch.float64), inv)
    return torch.cos(ang).repeat(1, 2), torch.sin(ang).repeat(1, 2)


def plain_rotate_half(x):
    """main_models_new.py:71-73 — (x1, x2) -> (-x2, x1), halves not interleaved."""
    x1, x2 = x.chunk(2, dim=-1)
    return torch.cat((-x2, x1), dim=-1)


def plain_apply_rope(x, cos, sin):
    """main_models_new.py:75-80 — x*cos + rotate_half(x)*sin; x is (T, heads, hd)."""
    c, s = cos.to(x.dtype).unsqueeze(1), sin.to(x.dtype).unsqueeze(1)
    return x * c + plain_rotate_half(x) * s


def plain_causal_attention(q, k, v, window=None, q_offset=0):
    """Dense softmax attention.  q (Tq, H, hd); k, v (Tk, KVH, hd); query head h uses
    kv head h // (H // KVH) (paged_attention_kernels.py:49, intradocatt_fwd_kernels.py:42).
    Scores q.k / sqrt(hd) (paged_attention_kernels.py:214); the query at position p sees
    keys 0..p (paged_attention_kernels.py:93-97).  ``window`` (engine option): only keys
    p-window+1..p.  ``q_offset``: position of the first query among the keys.
    """
    Tq, H, hd = q.shape
    Tk, KVH, _ = k.shape
    g = H // KVH
    kk = k.repeat_interleave(g, dim=1)
    vv = v.repeat_interleave(g, dim=1)
    s = torch.einsum("qhd,khd->hqk", q, kk) / math.sqrt(hd)
    qpos = torch.arange(Tq).unsqueeze(1) + q_offset
    kpos = torch.arange(Tk).unsqueeze(0)
    ok = kpos <= qpos
    if window is not None:
        ok = ok & (kpos > qpos - window)
    s = s.masked_fill(~ok.unsqueeze(0), float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hqk,khd->qhd", p, vv)


def plain_swiglu_ffn(x, w_gate, w_up, w_down):
    """main_models_new.py:44-60 — (silu(x W1) * (x W2)) W3, weights stored (in, out)."""
    return (torch.nn.functional.silu(x @ w_gate) * (x @ w_up)) @ w_down


def _kv_project(a, W, prefix, c):
    """main_models_new.py:104-106 — kv_proj output viewed (T, 2, KVH, hd): keys are the
    first half of the columns, values the second."""
    T = a.shape[0]
    kv = (a @ W[prefix + "att.kv_proj.weight"]).view(T, 2, c["num_kv_heads"], c["head_dim"])
    return kv[:, 0], kv[:, 1]


def plain_block(x, W, prefix, c, positions, window, shared_kv=None):
    """main_models_new.py:96-115 (attention half) and :139-148 (block).

    Returns the block output and the (rotated keys, values) it used, so that a later
    layer of the schedule can read them (engine option ``cache_source``).
    """
    T, d = x.shape
    H, hd = c["num_heads"], c["head_dim"]
    a = plain_rms_norm(x, W[prefix + "att.rms_norm_att.scale"], c["rms_norm_eps"])
    q = (a @ W[prefix + "att.q_proj.weight"]).view(T, H, hd)
    cos, sin = plain_rope_angles(positions, c["rope_theta"], hd)
    q = plain_apply_rope(q, cos, sin)
    if shared_kv is None:
        k, v = _kv_project(a, W, prefix, c)
        k = plain_apply_rope(k, cos, sin)
    else:
        k, v = shared_kv
    o = plain_causal_attention(q, k, v, window=window)
    x = x + o.reshape(T, H * hd) @ W[prefix + "att.linear_proj.weight"]
    f = plain_rms_norm(x, W[prefix + "rms_norm_ffn.scale"], c["rms_norm_eps"])
    x = x + plain_swiglu_ffn(f, W[prefix + "ffn.swig.linear1.weight"],
                             W[prefix + "ffn.swig.linear2.weight"], W[prefix + "ffn.fc.weight"])
    return x, (k, v)


def layer_window(c, layer_index):
    """Engine option: ``sliding_window`` applies to every layer (trunk layers are
    0..L-1, the block of MTP head i is layer L+i) except those named in
    ``full_attention_layers``."""
    w = c.get("sliding_window")
    if w is None:
        return None
    full = c.get("full_attention_layers") or []
    return None if layer_index in full else int(w)


def plain_trunk(c, W, ids):
    """main_models_new.py:197-202 — embedding, the blocks in schedule order, final norm.
    Returns rms_out(x) at every position, (T, d)."""
    ids = torch.as_tensor(ids, dtype=torch.long)
    T = ids.shape[0]
    pos = torch.arange(T)
    x = W["embedding.weight"][ids]
    order = c.get("layer_order") or list(range(c["num_layers"]))
    source = c.get("cache_source") or [None] * len(order)
    kept = []
    for e, layer in enumerate(order):
        shared = kept[source[e]] if source[e] is not None else None
        x, kv = plain_block(x, W, f"transformer_block_list.{layer}.", c, pos,
                            layer_window(c, layer), shared_kv=shared)
        kept.append(kv)
    return plain_rms_norm(x, W["rms_out.scale"], c["rms_norm_eps"])


def plain_mtp_head(c, W, i, h_prev, ids):
    """main_models_new.py:155-171 and the coverage rule of server.py:333-336.

    Head i at position p takes the previous stage's (already normalised) output at p
    and the embedding of token p+1+i, for p in [0, T-2-i]:
    u = cat[h_prev, rms_embed(E[tok])] @ Wp ; one block at RoPE position p over the
    head's own keys ; g = rms_out(u).  Returns g, (T-1-i, d).
    """
    ids = torch.as_tensor(ids, dtype=torch.long)
    T = ids.shape[0]
    n = max(0, T - 1 - i)
    pre = f"mtp_heads_list.{i}."
    if n == 0:
        return h_prev[:0]
    e = plain_rms_norm(W["embedding.weight"][ids[1 + i:1 + i + n]], W[pre + "rms_embed.scale"],
                       c["rms_norm_eps"])
    u = torch.cat([h_prev[:n], e], dim=-1) @ W[pre + "proj.weight"]
    u, _ = plain_block(u, W, pre + "trans_block.", c, torch.arange(n),
                       layer_window(c, c["num_layers"] + i))
    return plain_rms_norm(u, W[pre + "rms_out.scale"], c["rms_norm_eps"])


def plain_logits(c, W, h):
    """main_models_new.py:225-226 — h @ E^T; with ``tie_word_embeddings`` false (engine
    option) h @ lm_head^T instead."""
    out = W["embedding.weight"] if c["tie_word_embeddings"] else W["lm_head.weight"]
    return h @ out.T


def plain_forward(c, W, ids, mtp=True):
    """Logits of the main model at every position and of every MTP head at the
    positions it covers: {"main": (T, V), "mtp": [(T-1-i, V) for each head i]}."""
    h = plain_trunk(c, W, ids)
    out = {"main": plain_logits(c, W, h), "mtp": []}
    if mtp:
        prev = h
        for i in range(c["num_mtp_heads"]):
            prev = plain_mtp_head(c, W, i, prev, ids)
            out["mtp"].append(plain_logits(c, W, prev))
    return out


def plain_greedy(c, W, prompt, new_tokens):
    """Greedy continuation by recomputing the whole sequence for every token."""
    ids = list(prompt)
    for _ in range(new_tokens):
        h = plain_trunk(c, W, ids)
        ids.append(int(plain_logits(c, W, h[-1:]).argmax(-1)))
    return ids[len(prompt):]


# --------------------------------------------------------------------------------------
# sampling
# --------------------------------------------------------------------------------------

def plain_probs(logits, temperature, top_k=0, top_p=0.0, rep_penalty=1.0, ctx=()):
    """server.py:22-50 for one row: repetition penalty over the distinct context tokens
    (positive logits divided, others multiplied, :29-36), division by the temperature
    (:38), top-k by rank in one descending sort (:40-42), top-p removing entries whose
    preceding cumulative probability already exceeds p (:44-48), softmax (:50)."""
    x = logits.to(torch.float64).clone()
    if rep_penalty != 1.0:
        for t in set(int(t) for t in ctx):
            x[t] = x[t] / rep_penalty if x[t] > 0 else x[t] * rep_penalty
    x = x / temperature
    srt, idx = torch.sort(x, descending=True, stable=True)
    V = x.shape[0]
    k = top_k if top_k > 0 else V
    srt[k:] = float("-inf")
    pp = top_p if top_p > 0 else 2.0
    cum = torch.cumsum(torch.softmax(srt, -1), -1)
    remove = cum > pp
    remove[1:] = remove[:-1].clone()
    remove[0] = False
    srt[remove] = float("-inf")
    out = torch.full_like(x, float("-inf"))
    out[idx] = srt
    return torch.softmax(out, -1)
