"""The sampling kernel: probabilities against the plain implementation of upstream's
sampler (tests/plain_model.py: plain_probs), arg-max, determinism, and the distribution of
many draws."""
import pytest
import torch

import kernel_refs as ref
import plain_model

pytestmark = pytest.mark.gpu


def _ops():
    from tiny_inference_server_b200.kernels import ops
    ops.library()
    return ops


def _run(ops, logits, temps, top_ks, top_ps, pens, seen_lists, seeds, counters, want_probs=True):
    k, V = logits.shape
    words = (V + 31) // 32
    bitmap = torch.zeros(k, words, dtype=torch.int32)
    for r, toks in enumerate(seen_lists):
        if toks:
            ref.bitmap_set(bitmap[r], torch.tensor(toks))
    dev = "cuda"
    probs = torch.empty(k, V, device=dev) if want_probs else None
    out = torch.empty(k, dtype=torch.int32, device=dev)
    bm = bitmap.to(dev)
    ops.sample_rows(logits.to(dev), torch.tensor(temps, dtype=torch.float32, device=dev),
                    torch.tensor(top_ks, dtype=torch.int32, device=dev),
                    torch.tensor(top_ps, dtype=torch.float32, device=dev),
                    torch.tensor(pens, dtype=torch.float32, device=dev),
                    torch.arange(k, dtype=torch.int32, device=dev), bm,
                    torch.tensor(seeds, dtype=torch.int64, device=dev),
                    torch.tensor(counters, dtype=torch.int64, device=dev), out, probs)
    return out.cpu(), (probs.cpu() if want_probs else None), bm.cpu()


@pytest.fixture
def stage_limit():
    """Sets how much of a row a CTA keeps in shared memory; the device's own limit again afterwards."""
    ops = _ops()
    yield ops.sample_stage_limit
    ops.sample_stage_limit(-1)


# (vocabulary, entries of a row a CTA may keep): one CTA a row; eight with a share each; shares of 76 entries
# in four CTAs; no share kept at all (every pass reads the logits), in one CTA and in eight
@pytest.mark.parametrize("V,limit", [(6, -1), (100, -1), (301, -1), (49152, -1), (301, 80), (100, 0), (8193, 0),
                                     (128256, -1)])
def test_probabilities_match_upstream_formulas(V, limit, stage_limit):
    ops = _ops()
    stage_limit(limit)
    g = torch.Generator().manual_seed(0)
    settings = [(1.0, 0, 0.0, 1.0), (0.7, 0, 0.0, 1.0), (1.0, 3, 0.0, 1.0), (1.0, 0, 0.9, 1.0),
                (0.9, 50, 0.95, 1.1), (1.3, 5, 0.5, 1.3), (1.0, 0, 0.0, 2.0), (0.5, 2, 0.3, 1.0)]
    k = len(settings)
    logits = torch.randn(k, V, generator=g) * 3
    seen = [torch.randint(0, V, (min(V, 20),), generator=g).tolist() for _ in range(k)]
    out, probs, _ = _run(ops, logits, [s[0] for s in settings], [s[1] for s in settings],
                         [s[2] for s in settings], [s[3] for s in settings], seen, [1] * k, [0] * k)
    for r, (t, tk, tp, pen) in enumerate(settings):
        want = plain_model.plain_probs(logits[r], t, tk, tp, pen, seen[r]).float()
        torch.testing.assert_close(probs[r], want, rtol=1e-4, atol=1e-6)
        assert probs[r, out[r]] > 0


def test_greedy_takes_lowest_index_of_the_maximum_and_applies_penalty():
    ops = _ops()
    V = 100
    lg = torch.zeros(3, V)
    lg[0, 5] = 5.0
    lg[0, 7] = 4.9
    lg[1] = lg[0]
    lg[2, 40] = 2.0
    lg[2, 60] = 2.0
    out, _, bm = _run(ops, lg, [0.0, 0.0, 1.0], [0, 0, 1], [0.0] * 3, [1.0, 2.0, 1.0], [[], [5], []], [0] * 3,
                      [0] * 3)
    # upstream's check (test_server.py:120-122): the penalty pushes token 5 below token 7
    assert out.tolist() == [5, 7, 40]


@pytest.mark.parametrize("k,V", [(1, 49152), (8, 8193), (3, 1025), (40, 5000), (200, 3000), (5, 1024)])
def test_arg_max_over_the_ctas_of_a_row(k, V):
    """The first pass runs over several CTAs a row (fewer the more rows there are), in runs of 1024 entries:
    the maximum in every run in turn, and equal maxima in runs of different CTAs (lowest index wins); the
    probabilities of a sampled row need the maximum of the whole row too."""
    ops = _ops()
    g = torch.Generator().manual_seed(k * 7 + V)
    logits = torch.randn(k, V, generator=g)
    want = []
    for r in range(k):
        a = (r * 1024 + 17 * r + 5) % V             # a run further on for every row
        b = (a + 3 * 1024 + 1) % V                  # the same value in another run
        logits[r, a] = 9.0
        if r % 2:
            logits[r, b] = 9.0
            want.append(min(a, b))
        else:
            want.append(a)
    out, _, _ = _run(ops, logits, [0.0] * k, [0] * k, [0.0] * k, [1.0] * k, [[]] * k, [0] * k, [0] * k, want_probs=False)
    assert out.tolist() == want
    out, probs, _ = _run(ops, logits, [1.0] * k, [0] * k, [0.0] * k, [1.0] * k, [[]] * k, [3] * k, list(range(k)))
    torch.testing.assert_close(probs, torch.softmax(logits, -1), rtol=1e-4, atol=1e-7)


@pytest.mark.parametrize("V,limit", [(49152, -1), (8193, -1), (301, 80), (5000, 0), (5000, 700)])
def test_draws_lie_in_their_interval_of_the_cdf_with_several_ctas_a_row(V, limit, stage_limit):
    """Rows of every kind of setting, several draws each: the uniform number of (seed, counter) lies inside the
    drawn token's own interval of the reference CDF (widened by float32 rounding of the sums, which the kernel
    adds up in another order), whichever CTA of the row holds the token."""
    ops = _ops()
    stage_limit(limit)
    g = torch.Generator().manual_seed(V + limit)
    settings = [(1.0, 0, 0.0, 1.0), (1.0, 40, 0.0, 1.0), (1.0, 0, 0.9, 1.0), (0.8, 50, 0.95, 1.1)]
    draws = 6
    k = len(settings) * draws
    logits = (torch.randn(len(settings), V, generator=g) * 2).repeat_interleave(draws, 0)
    rows = [s for s in settings for _ in range(draws)]
    seen = [[1, V - 1]] * k
    seeds, counters = [5] * k, list(range(k))
    out, _, _ = _run(ops, logits, [s[0] for s in rows], [s[1] for s in rows], [s[2] for s in rows],
                     [s[3] for s in rows], seen, seeds, counters, want_probs=False)
    owners = set()
    for r, (t, tk, tp, pen) in enumerate(rows):
        p = ref.row_probs(logits[r], t, tk, tp, pen, seen[r])
        u = (ref._philox_u32(seeds[r], counters[r]) >> 8) / 16777216.0
        cum = torch.cumsum(p, -1)
        tok = int(out[r])
        lo = float(cum[tok - 1]) if tok > 0 else 0.0
        assert float(p[tok]) > 0 and lo - 2e-5 <= u * float(cum[-1]) <= float(cum[tok]) + 2e-5, \
            f"row {r} {rows[r]}: token {tok} drawn for u={u}, its interval is [{lo}, {float(cum[tok])}]"
        owners.add(tok * 8 // V)
    assert len(owners) > 2 or V < 1000          # the tokens came from several parts of the row


@pytest.mark.parametrize("V,limit", [(5000, -1), (300, 40), (49152, -1)])
def test_equal_values_at_a_threshold_are_all_kept(V, limit, stage_limit):
    """Logits on a grid of quarter steps (hundreds of equal values): the k-th largest value and the value at which
    the cumulative probability passes p are shared by many entries, all of which stay (the radix passes end early
    when a whole bin is wanted, or run to the last bit: both must give the same set)."""
    ops = _ops()
    stage_limit(limit)
    g = torch.Generator().manual_seed(V)
    settings = [(1.0, 3, 0.0), (1.0, 40, 0.0), (1.0, 0, 0.5), (1.0, 200, 0.9), (1.0, 1000, 0.0), (1.0, V - 1, 0.0)]
    k = len(settings)
    logits = (torch.randn(k, V, generator=g) * 2).mul(4).round().div(4)
    out, probs, _ = _run(ops, logits, [s[0] for s in settings], [s[1] for s in settings], [s[2] for s in settings],
                         [1.0] * k, [[]] * k, [1] * k, [0] * k)
    for r, (t, tk, tp) in enumerate(settings):
        want = ref.row_probs(logits[r], t, tk, tp, 1.0, []).float()
        assert int((probs[r] > 0).sum()) == int((want > 0).sum()), settings[r]
        torch.testing.assert_close(probs[r], want, rtol=1e-4, atol=1e-7)
        assert probs[r, out[r]] > 0


def test_same_seed_same_token_and_seen_bitmap_grows():
    ops = _ops()
    g = torch.Generator().manual_seed(1)
    V = 1000
    logits = torch.randn(4, V, generator=g)
    a, _, bm = _run(ops, logits, [1.0] * 4, [0] * 4, [0.0] * 4, [1.2] * 4, [[1]] * 4, [11, 11, 12, 11], [0, 0, 0, 1])
    b, _, _ = _run(ops, logits, [1.0] * 4, [0] * 4, [0.0] * 4, [1.2] * 4, [[1]] * 4, [11, 11, 12, 11], [0, 0, 0, 1])
    assert a.tolist() == b.tolist()
    for r in range(4):
        t = int(a[r])
        assert (int(bm[r, t >> 5]) >> (t & 31)) & 1
    # the reference sampler draws with the same generator and inverse CDF
    want = torch.empty(4, dtype=torch.int32)
    bitmap = torch.zeros(4, (V + 31) // 32, dtype=torch.int32)
    for r in range(4):
        ref.bitmap_set(bitmap[r], torch.tensor([1]))
    ref.sample_rows(logits, [1.0] * 4, [0] * 4, [0.0] * 4, [1.2] * 4, list(range(4)), bitmap, [11, 11, 12, 11],
                    [0, 0, 0, 1], want)
    # Every drawn token is the reference's, or its neighbour in the CDF where the uniform number falls
    # within float32 rounding of the edge between the two (the kernel adds up the CDF in float32 in another
    # order than the float64 reference): the number must lie inside the drawn token's own interval of the
    # reference CDF, widened by 1e-5 — a wrong edge rule (>= for >, an interval shifted by one token) puts it
    # a whole probability mass outside.
    for r, (seed, counter) in enumerate(zip([11, 11, 12, 11], [0, 0, 0, 1])):
        p = ref.row_probs(logits[r], 1.0, 0, 0.0, 1.2, [1])
        u = (ref._philox_u32(seed, counter) >> 8) / 16777216.0
        cum = torch.cumsum(p, -1)
        t = int(a[r])
        lo = float(cum[t - 1]) if t > 0 else 0.0
        assert float(p[t]) > 0 and lo - 1e-5 <= u * float(cum[-1]) <= float(cum[t]) + 1e-5, \
            f"row {r}: token {t} drawn for u={u}, its interval is [{lo}, {float(cum[t])}]"
        assert float(p[t]) > 1e-4 or t == int(want[r])     # an interval narrower than the margin proves nothing


@pytest.mark.parametrize("setting", [(1.0, 0, 0.0), (1.0, 3, 0.9), (0.8, 0, 0.7)])
def test_distribution_of_many_draws(setting):
    """4096 draws from one row of six logits (upstream's distribution test uses vocabulary 6,
    test_server.py:124-141): total variation to the exact probabilities stays small."""
    ops = _ops()
    t, tk, tp = setting
    V, N = 6, 4096
    row = torch.tensor([1.0, 0.5, -0.3, 2.0, 0.0, 1.5])
    logits = row.repeat(N, 1)
    out, _, _ = _run(ops, logits, [t] * N, [tk] * N, [tp] * N, [1.0] * N, [[]] * N, [5] * N, list(range(N)),
                     want_probs=False)
    hist = torch.bincount(out.long(), minlength=V).double() / N
    want = plain_model.plain_probs(row, t, tk, tp)
    tv = 0.5 * (hist - want).abs().sum()
    assert tv < 0.03, f"total variation {tv}"
