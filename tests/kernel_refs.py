"""Plain PyTorch references of the device operations, one per kernel, with the
signatures of ``tiny_inference_server_b200.kernels.ops``.

They serve two purposes: the GPU tests compare each CUDA kernel alone with its reference
here (at sizes other than the engine's), and the CPU tests put them in place of the
kernels (``install``) so that the cache manager, the step function, the scheduler and
trace replay can be checked where there is no GPU.  They are slow and obvious on
purpose; nothing of the product imports this file.
"""
from __future__ import annotations

import math
from typing import Optional

import torch


def _row_factor(scaled):
    """The norm's factor of each row from the partial sums of squares: "l2_eps": sqrt(width) / (||row|| + eps);
    "mean_eps": 1 / sqrt(mean of squares + eps)."""
    d = scaled.rows.shape[1]
    s = scaled.parts.sum(-1, keepdim=True)
    if scaled.kind == "mean_eps":
        return 1.0 / torch.sqrt(s / d + scaled.eps)
    return math.sqrt(d) / (s.sqrt() + scaled.eps)


def scaled_rows_dense(scaled):
    return (scaled.rows.to(torch.float32) * _row_factor(scaled)).to(scaled.rows.dtype)


def gemm(a, w, out=None, sink=None):
    """``a`` may be ``ops.ScaledRows`` (the product is multiplied by each row's factor afterwards); with a
    ``sink`` of matching shape and few bfloat16 rows the product is added to the stream there and the
    stream times the next norm's weight comes back with partial sums of squares by strip of 64 columns."""
    from tiny_inference_server_b200.kernels import ops
    factor = None
    if isinstance(a, ops.ScaledRows):
        factor, a = _row_factor(a), a.rows
    r = a.to(torch.float32) @ w.to(torch.float32)
    if factor is not None:
        r = r * factor
    if (sink is not None and out is None and a.dtype == torch.bfloat16 and a.shape[0] <= ops.SKINNY_MAX_ROWS
            and tuple(sink.values.shape) == tuple(r.shape)):
        sink.values += r
        n, d = r.shape
        strips = -(-d // 64)
        sq = torch.zeros((n, strips * 64), dtype=torch.float32)
        sq[:, :d] = sink.values.pow(2)
        return ops.ScaledRows((sink.values * sink.weight).to(a.dtype), sq.reshape(n, strips, 64).sum(-1), sink.eps, sink.norm,
                              sink.kind)
    r = r.to(a.dtype)
    if out is not None:
        out.copy_(r)
        return out
    return r


def gemm_f32_out(a, w):
    return a.to(torch.float32) @ w.to(torch.float32)


def embed_rows(table, tokens, out):
    out.copy_(table[tokens.long()].to(torch.float32))
    return out


def add_rmsnorm(residual, delta, scale, eps, out):
    if delta is not None:
        residual += delta.to(torch.float32)
    if out is None:
        return None
    d = residual.shape[-1]
    norm = residual.pow(2).sum(-1, keepdim=True).sqrt()
    out.copy_((residual * math.sqrt(d) / (norm + eps) * scale).to(out.dtype))
    return out


def residual_add(residual, delta):
    residual += delta.to(torch.float32)
    return residual


def _rotate(x, cos, sin, interleaved):
    """x (heads, hd) float32; cos, sin (rot/2,)."""
    rot = 2 * cos.shape[0]
    y = x.clone()
    if interleaved:
        a, b = x[:, 0:rot:2], x[:, 1:rot:2]
        y[:, 0:rot:2] = a * cos - b * sin
        y[:, 1:rot:2] = b * cos + a * sin
    else:
        h = rot // 2
        a, b = x[:, :h], x[:, h:rot]
        y[:, :h] = a * cos - b * sin
        y[:, h:rot] = b * cos + a * sin
    return y


def _chunk_places(nch, positions):
    """physical chunk of logical chunk c for rows at ``positions``: (L, nch).  Rows of a multiple
    of eight chunks: c XOR (position mod 8); other rows: (c + position) mod chunks."""
    c = torch.arange(nch)[None, :]
    pos = torch.as_tensor(positions).reshape(-1, 1)
    return (c ^ (pos & 7)) if nch % 8 == 0 else (c + pos) % nch


def cache_row(x, pos):
    """The cache's row format: a row of keys or values (last axis: head size) is stored as
    16-byte chunks permuted by the position."""
    n = 16 // x.element_size()
    hd = x.shape[-1]
    place = _chunk_places(hd // n, [pos])[0]
    chunks = x.reshape(*x.shape[:-1], hd // n, n)
    out = torch.empty_like(chunks)
    out[..., place, :] = chunks
    return out.reshape(x.shape)


def cache_row_inverse(x, pos):
    n = 16 // x.element_size()
    hd = x.shape[-1]
    place = _chunk_places(hd // n, [pos])[0]
    return x.reshape(*x.shape[:-1], hd // n, n)[..., place, :].reshape(x.shape)


def rope_kv_write(qkv, positions, row_slot, cos, sin, plane, block_table, num_heads, kv_heads, head_dim,
                  page_size, fault, interleaved=False, write_kv=True):
    n = qkv.shape[0]
    hq, hkv = num_heads * head_dim, kv_heads * head_dim
    for r in range(n):
        slot = int(row_slot[r])
        if slot < 0:
            continue
        pos = int(positions[r])
        c, s = cos[pos], sin[pos]
        q = qkv[r, :hq].to(torch.float32).view(num_heads, head_dim)
        qkv[r, :hq] = _rotate(q, c, s, interleaved).reshape(-1).to(qkv.dtype)
        if not (write_kv and plane is not None):
            continue
        page = int(block_table[slot, pos // page_size])
        if page < 0 or page >= plane.shape[0]:
            fault[0] = 1
            continue
        k = qkv[r, hq:hq + hkv].to(torch.float32).view(kv_heads, head_dim)
        v = qkv[r, hq + hkv:hq + 2 * hkv].view(kv_heads, head_dim)
        plane[page, 0, :, pos % page_size, :] = cache_row(_rotate(k, c, s, interleaved).to(plane.dtype), pos)
        plane[page, 1, :, pos % page_size, :] = cache_row(v.to(plane.dtype), pos)


def gather_kv(plane, block_table, slot, lo, hi, page_size):
    """Keys and values lo..hi-1 of a slot: (hi-lo, KVH, hd) each, float32."""
    idx = torch.arange(lo, hi)
    pages = block_table[slot, (idx // page_size)].long()
    k = _unrotate_rows(plane[pages, 0, :, idx % page_size, :], idx)
    v = _unrotate_rows(plane[pages, 1, :, idx % page_size, :], idx)
    return k.to(torch.float32), v.to(torch.float32)


def _unrotate_rows(x, positions):
    """x (L, KVH, hd) as stored, row i belonging to positions[i]: back to logical order."""
    n = 16 // x.element_size()
    L, kvh, hd = x.shape
    nch = hd // n
    chunks = x.reshape(L, kvh, nch, n).permute(0, 2, 1, 3)                       # (L, nch, KVH, n)
    phys = _chunk_places(nch, positions)                                         # logical c -> physical chunk
    out = chunks[torch.arange(L)[:, None], phys]                                 # (L, nch, KVH, n)
    return out.permute(0, 2, 1, 3).reshape(L, kvh, hd)


def rotary_fusable(q, step, num_heads, kv_heads, head_dim):
    """On the CPU every decode step takes the path where attention does the rotary encoding and the
    cache write itself, so that its plumbing runs in the CPU tests too."""
    return step is not None and getattr(step, "decode_only", False)


def paged_attention(q, out, plane, block_table, positions, row_slot, num_heads, kv_heads, head_dim, page_size,
                    window, fault, step=None, rotary=None, write_kv=True):
    if rotary is not None:
        rope_kv_write(q, positions, row_slot, rotary[0], rotary[1], plane, block_table, num_heads, kv_heads, head_dim,
                      page_size, fault, write_kv=write_kv)
    n = q.shape[0]
    g = num_heads // kv_heads
    hq = num_heads * head_dim
    for r in range(n):
        slot = int(row_slot[r])
        if slot < 0:
            out[r] = 0
            continue
        pos = int(positions[r])
        hi = pos + 1
        lo = max(0, hi - window) if window else 0
        k, v = gather_kv(plane, block_table, slot, lo, hi, page_size)
        k = k.repeat_interleave(g, dim=1)
        v = v.repeat_interleave(g, dim=1)
        qq = q[r, :hq].to(torch.float32).view(num_heads, head_dim)
        s = torch.einsum("hd,khd->hk", qq, k) / math.sqrt(head_dim)
        p = torch.softmax(s, dim=-1)
        out[r] = torch.einsum("hk,khd->hd", p, v).reshape(-1).to(out.dtype)
    return out


def swiglu(gu, out, block=None):
    f = out.shape[1]
    block = block or f
    both = gu.to(torch.float32).reshape(gu.shape[0], f // block, 2, block)
    g = both[:, :, 0, :].reshape(-1, f)
    u = both[:, :, 1, :].reshape(-1, f)
    out.copy_((g / (1 + torch.exp(-g)) * u).to(out.dtype))
    return out


def gemm_swiglu(a, w_gu, hidden, block):
    gu = gemm(a, w_gu)
    return swiglu(gu, torch.empty((a.shape[0], hidden), dtype=a.dtype), block)


def mtp_input(h_prev, state, row_slot, row_last, tokens, table, scale, eps, out):
    n, d = h_prev.shape
    new_state = {}
    for r in range(n):
        slot = int(row_slot[r])
        if slot < 0:
            continue
        first = r == 0 or int(row_slot[r - 1]) != slot
        if first:
            out[r, :d] = state[slot]
            new_state[slot] = h_prev[int(row_last[r])].clone()
        else:
            out[r, :d] = h_prev[r - 1]
        e = table[int(tokens[r])].to(torch.float32)
        norm = e.pow(2).sum().sqrt()
        out[r, d:] = (e * math.sqrt(d) / (norm + eps) * scale).to(out.dtype)
    for slot, row in new_state.items():
        state[slot] = row
    return out


def _philox_u32(seed: int, counter: int) -> int:
    m0, m1 = 0xD2511F53, 0xCD9E8D57
    c = [counter & 0xFFFFFFFF, (counter >> 32) & 0xFFFFFFFF, 0, 0]
    k0, k1 = seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF
    for _ in range(10):
        p0, p1 = m0 * c[0], m1 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k0) & 0xFFFFFFFF, p1 & 0xFFFFFFFF,
             ((p0 >> 32) ^ c[3] ^ k1) & 0xFFFFFFFF, p0 & 0xFFFFFFFF]
        k0 = (k0 + 0x9E3779B9) & 0xFFFFFFFF
        k1 = (k1 + 0xBB67AE85) & 0xFFFFFFFF
    return c[0]


def row_probs(logits_row, temp, top_k, top_p, penalty, seen_tokens):
    """Probabilities of one row as the sampling kernel defines them: all entries equal to a
    threshold value are kept."""
    x = logits_row.to(torch.float64).clone()
    if penalty != 1.0 and len(seen_tokens):
        idx = torch.tensor(sorted(set(int(t) for t in seen_tokens)), dtype=torch.long)
        x[idx] = torch.where(x[idx] > 0, x[idx] / penalty, x[idx] * penalty)
    x = x / temp
    v = x.shape[0]
    keep = torch.ones(v, dtype=torch.bool)
    if 0 < top_k < v:
        thr = torch.sort(x, descending=True).values[top_k - 1]
        keep &= x >= thr
    if 0 < top_p < 1:
        xs = torch.where(keep, x, torch.full_like(x, float("-inf")))
        p = torch.softmax(xs, -1)
        srt, _ = torch.sort(p, descending=True)
        cum = torch.cumsum(srt, -1)
        first_over = int((cum > top_p).nonzero()[0]) if bool((cum > top_p).any()) else v - 1
        keep &= p >= srt[first_over]
    xs = torch.where(keep, x, torch.full_like(x, float("-inf")))
    return torch.softmax(xs, -1)


def sample_rows(logits, temps, top_ks, top_ps, penalties, slots, seen_bitmap, seeds, counters, out_tokens,
                probs_out=None):
    k, v = logits.shape
    for r in range(k):
        temp, top_k = float(temps[r]), int(top_ks[r])
        slot = int(slots[r]) if slots is not None else -1
        seen = []
        if slot >= 0 and seen_bitmap is not None:
            words = seen_bitmap[slot]
            seen = [i for i in range(v) if (int(words[i >> 5]) >> (i & 31)) & 1]
        pen = float(penalties[r])
        greedy = not (temp > 0) or top_k == 1
        if greedy:
            x = logits[r].to(torch.float64).clone()
            if pen != 1.0 and seen:
                idx = torch.tensor(seen, dtype=torch.long)
                x[idx] = torch.where(x[idx] > 0, x[idx] / pen, x[idx] * pen)
            tok = int(torch.argmax(x))
            p = torch.zeros(v, dtype=torch.float64)
            p[tok] = 1
        else:
            p = row_probs(logits[r], temp, top_k, float(top_ps[r]), pen, seen)
            u = (_philox_u32(int(seeds[r]), int(counters[r])) >> 8) / 16777216.0
            cum = torch.cumsum(p, -1)
            over = (cum > u * float(cum[-1])) & (p > 0)
            tok = int(over.nonzero()[0]) if bool(over.any()) else int((p > 0).nonzero()[-1])
        out_tokens[r] = tok
        if probs_out is not None:
            probs_out[r] = p.to(torch.float32)
        if slot >= 0 and seen_bitmap is not None:
            w = int(seen_bitmap[slot, tok >> 5]) & 0xFFFFFFFF
            w |= 1 << (tok & 31)
            seen_bitmap[slot, tok >> 5] = w - (1 << 32) if w >= (1 << 31) else w
    return out_tokens


def bitmap_set(bitmap_row, tokens):
    for t in tokens.tolist():
        w = int(bitmap_row[t >> 5]) & 0xFFFFFFFF
        w |= 1 << (t & 31)
        bitmap_row[t >> 5] = w - (1 << 32) if w >= (1 << 31) else w


_NAMES = ["rotary_fusable", "gemm", "gemm_f32_out", "gemm_swiglu", "embed_rows", "add_rmsnorm", "residual_add", "rope_kv_write",
          "paged_attention", "swiglu", "mtp_input", "sample_rows", "bitmap_set"]


def install(monkeypatch) -> None:
    """Put the references in place of the CUDA operations (CPU tests only)."""
    from tiny_inference_server_b200.kernels import ops

    g = globals()
    for name in _NAMES:
        monkeypatch.setattr(ops, name, g[name])
    monkeypatch.setattr(ops.ScaledRows, "dense", scaled_rows_dense)
