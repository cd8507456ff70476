"""Builds traces (lists of step objects for trace replay) that feed the same requests in
different ways, and gathers what a replay wrote back into per-request logits."""
from __future__ import annotations

import os
from typing import Dict, List, Sequence

import numpy as np


def _step(i, entries, end=()):
    return {"step": i, "entries": entries, "end": list(end)}


def trace_whole(seqs: Dict[str, Sequence[int]]):
    """Each request alone and whole; logits wanted everywhere."""
    steps = []
    for rid, toks in seqs.items():
        steps.append(_step(len(steps), [{"id": rid, "tokens": list(toks), "want": list(range(len(toks)))}], [rid]))
    return steps


def trace_tail(seqs: Dict[str, Sequence[int]], tail: int = 32):
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    steps = []
    for rid, toks in seqs.items():
        toks = list(toks)
        head = max(0, len(toks) - tail)
        if head:
            steps.append(_step(len(steps), [{"id": rid, "tokens": toks[:head], "want": list(range(head))}]))
        for p in range(head, len(toks)):
            steps.append(_step(len(steps), [{"id": rid, "tokens": [toks[p]], "want": [0]}],
                               [rid] if p == len(toks) - 1 else []))
    return steps


def trace_chunks(seqs: Dict[str, Sequence[int]], sizes=(7, 2, 16, 3, 2, 1, 5, 2, 9)):
    """Portions of changing size, down to two tokens and one."""
    steps = []
    for rid, toks in seqs.items():
        toks = list(toks)
        p, k = 0, 0
        while p < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - p)
            k += 1
            steps.append(_step(len(steps), [{"id": rid, "tokens": toks[p:p + n], "want": list(range(n))}],
                               [rid] if p + n == len(toks) else []))
            p += n
    return steps


def trace_mixed(seqs: Dict[str, Sequence[int]], max_live: int = 4, prefill_sizes=(5, 2, 11, 3), decode_from=0.6,
                skip_every: int = 5):
    """Up to ``max_live`` requests at a time: each is first fed in portions of changing size,
    then (from ``decode_from`` of its length on) one token a step, so that portions of some
    stand beside single tokens of others.  Now and then a request is left out of a step.
    Requests end as they finish and new ones take their place, so pages are used again."""
    pending = list(seqs.items())
    live = []          # [rid, toks, fed, k]
    steps = []
    tick = 0
    while pending or live:
        while pending and len(live) < max_live:
            rid, toks = pending.pop(0)
            live.append([rid, list(toks), 0, 0])
        entries, end = [], []
        for j, item in enumerate(live):
            rid, toks, fed, k = item
            tick += 1
            if skip_every and tick % skip_every == 0 and len(live) > 1:
                continue       # left out of this step, goes on later
            if fed < int(len(toks) * decode_from):
                n = min(prefill_sizes[(k + j) % len(prefill_sizes)], len(toks) - fed)
            else:
                n = 1
            entries.append({"id": rid, "tokens": toks[fed:fed + n], "want": list(range(n))})
            item[2] += n
            item[3] += 1
            if item[2] == len(toks):
                end.append(rid)
        if entries:
            steps.append(_step(len(steps), entries, end))
        live = [it for it in live if it[2] < len(it[1])]
    return steps


def max_live_tokens(steps, round_to: int = 64) -> int:
    """The most tokens live requests hold at any time, each rounded up to ``round_to``."""
    held: Dict[str, int] = {}
    best = 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        best = max(best, sum((n + round_to - 1) // round_to * round_to for n in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return best


def gather(steps, out_dir: str, vocab: int, suffix: str = "f32") -> Dict[str, Dict[int, np.ndarray]]:
    """{request: {position: logits}} from the files a replay wrote."""
    pos: Dict[str, int] = {}
    out: Dict[str, Dict[int, np.ndarray]] = {}
    for s in steps:
        wanted = sum(len(e["want"]) for e in s["entries"])
        arr = None
        if wanted:
            path = os.path.join(out_dir, f"{s['step']}.{suffix}")
            arr = np.fromfile(path, dtype="<f4").reshape(wanted, vocab)
        row = 0
        for e in s["entries"]:
            start = pos.get(e["id"], 0)
            for w in e["want"]:
                out.setdefault(e["id"], {})[start + w] = arr[row]
                row += 1
            pos[e["id"]] = start + len(e["tokens"])
        for rid in s["end"]:
            pos.pop(rid, None)
    return out
