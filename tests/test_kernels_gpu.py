"""Each CUDA kernel alone against its plain PyTorch reference (tests/kernel_refs.py), in
float32 and bfloat16, at sizes other than the engine's tiny models: widths and
vocabularies that are no power of two, head sizes in steps of 16, odd numbers of heads
and groups, scattered pages, padding rows."""
import math

import pytest
import torch

import kernel_refs as ref

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def _ops():
    from tiny_inference_server_b200.kernels import ops
    ops.library()
    return ops


def _tol(dtype):
    return dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)


def _rand(shape, dtype, gen, scale=1.0):
    return (torch.randn(shape, generator=gen, dtype=torch.float32) * scale).to(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,d,V", [(5, 72, 301), (33, 1536, 1000), (2, 8200, 77)])
def test_embed_rows(dtype, n, d, V):
    ops = _ops()
    g = torch.Generator().manual_seed(0)
    table = _rand((V, d), dtype, g)
    tokens = torch.randint(0, V, (n,), generator=g, dtype=torch.int32)
    want = ref.embed_rows(table, tokens, torch.empty(n, d))
    got = ops.embed_rows(table.cuda(), tokens.cuda(), torch.empty(n, d, device="cuda"))
    torch.testing.assert_close(got.cpu(), want, rtol=0, atol=0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,d", [(1, 48), (7, 120), (19, 1536), (3, 4100), (2, 16384), (1024, 1536), (1203, 120), (1030, 2048),
                                 (1025, 264), (1026, 2056), (1100, 8)])
@pytest.mark.parametrize("with_delta", [False, True])
def test_add_rmsnorm(dtype, n, d, with_delta):
    ops = _ops()
    g = torch.Generator().manual_seed(1)
    res = torch.randn(n, d, generator=g) * 3
    delta = _rand((n, d), dtype, g) if with_delta else None
    scale = 1 + 0.1 * torch.randn(d, generator=g)
    eps = 1e-3
    res_ref = res.clone()
    want = ref.add_rmsnorm(res_ref, delta, scale, eps, torch.empty(n, d, dtype=dtype))
    res_dev = res.cuda()
    got = ops.add_rmsnorm(res_dev, None if delta is None else delta.cuda(), scale.cuda(), eps,
                          torch.empty(n, d, dtype=dtype, device="cuda"))
    torch.testing.assert_close(res_dev.cpu(), res_ref, rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(got.cpu().float(), want.float(), **_tol(dtype))


def test_add_rmsnorm_eps_is_added_to_the_norm():
    """With a large eps the two forms of RMSNorm differ; the kernel follows
    x*sqrt(d)/(||x||+eps), not x*rsqrt(mean(x^2)+eps)."""
    ops = _ops()
    d = 64
    x = torch.full((1, d), 0.5)
    scale = torch.ones(d)
    eps = 2.0
    got = ops.add_rmsnorm(x.cuda(), None, scale.cuda(), eps, torch.empty(1, d, device="cuda")).cpu()
    want = x * math.sqrt(d) / (x.norm() + eps)
    other = x * torch.rsqrt((x * x).mean() + eps)
    torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-6)
    assert (got - other).abs().max() > 0.05


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,F,block", [(3, 200, None), (17, 4096, None), (1, 10, None), (5, 352, 32), (9, 200, 5)])
def test_swiglu(dtype, n, F, block):
    ops = _ops()
    g = torch.Generator().manual_seed(2)
    gu = _rand((n, 2 * F), dtype, g, 2.0)
    want = ref.swiglu(gu, torch.empty(n, F, dtype=dtype), block)
    got = ops.swiglu(gu.cuda(), torch.empty(n, F, dtype=dtype, device="cuda"), block)
    torch.testing.assert_close(got.cpu().float(), want.float(), **_tol(dtype))


@pytest.mark.parametrize("kernel", ["boxes", "ring"])
@pytest.mark.parametrize("n", [1, 3, 8, 16, 17, 33, 64])
@pytest.mark.parametrize("K,N", [(1536, 2304), (128, 64), (200, 120), (4096, 1536), (72, 8), (1000, 1096),
                                 (8192, 200)])
def test_skinny_gemm(n, K, N, kernel, monkeypatch):
    """The weight-streaming products for few rows (a producer warp bringing a CTA's whole share of the weights
    as boxes of the TMA engine — K of 8192 over eight CTAs takes two rounds of boxes —; or the weights copied
    by all threads into a ring), for every split of K over a cluster."""
    ops = _ops()
    tma = kernel != "ring"
    monkeypatch.setattr(ops, "STREAM_GEMM", tma)
    monkeypatch.setattr(ops, "STREAM_MIN_KC", 0)           # every product that fits goes to the boxes
    monkeypatch.setattr(ops, "STREAM_MAX_KC", 1 << 30)
    monkeypatch.setattr(ops, "STREAM_MAX_CTAS", 1 << 30)
    monkeypatch.setattr(ops, "STREAM_MAX_ROWS", 64)
    before = ops.calls["gemm_stream"]
    g = torch.Generator().manual_seed(12)
    a = _rand((n, K), torch.bfloat16, g)
    w = _rand((K, N), torch.bfloat16, g, 0.05)
    want = (a.double() @ w.double())
    for ksplit in (None, 1, 2, 4, 8):
        got = ops.gemm_skinny(a.cuda(), w.cuda(), ksplit=ksplit)
        assert got.shape == (n, N) and got.dtype == torch.bfloat16
        torch.testing.assert_close(got.cpu().double(), want, rtol=2e-2, atol=2e-2)
    # a weight matrix that is a column slice of a wider one (row stride larger than its width)
    wide = _rand((K, N + 64), torch.bfloat16, g, 0.05).cuda()
    got = ops.gemm_skinny(a.cuda(), wide[:, :N])
    torch.testing.assert_close(got.cpu().double(), a.double() @ wide[:, :N].cpu().double(), rtol=2e-2, atol=2e-2)
    fits = sum(ops._stream_fits(n, K, ks or ops._ksplit(N, K)) for ks in (None, 1, 2, 4, 8, None))
    assert ops.calls["gemm_stream"] - before == (fits if tma else 0) and fits >= 2
    if tma and ops._tc_fault is not None:
        assert int(ops._tc_fault[0]) == 0, "a wait inside the kernel ran out"


@pytest.mark.parametrize("n", [1, 3, 8, 16, 17, 33, 64])
@pytest.mark.parametrize("K,N", [(1536, 2304), (128, 64), (200, 120), (4096, 1536), (72, 8), (1000, 1096), (8192, 200)])
def test_tcgen05_gemm_with_swapped_operands(n, K, N):
    """Few rows on the tcgen05 tensor cores: 128 columns of the weights are the rows of the tile, the rows of x its
    narrow side; every split of K over a cluster; ragged N and K (zeros from the TMA engine); a weight matrix that is
    a column slice of a wider one; the bounded waits must not have run out."""
    ops = _ops()
    g = torch.Generator().manual_seed(61)
    a = _rand((n, K), torch.bfloat16, g)
    w = _rand((K, N), torch.bfloat16, g, 0.05)
    want = (a.double() @ w.double())
    for ksplit in (None, 1, 2, 4, 8):
        got = ops.gemm_swap(a.cuda(), w.cuda(), ksplit=ksplit)
        assert got.shape == (n, N) and got.dtype == torch.bfloat16
        torch.testing.assert_close(got.cpu().double(), want, rtol=2e-2, atol=2e-2)
    wide = _rand((K, N + 64), torch.bfloat16, g, 0.05).cuda()
    got = ops.gemm_swap(a.cuda(), wide[:, :N])
    torch.testing.assert_close(got.cpu().double(), a.double() @ wide[:, :N].cpu().double(), rtol=2e-2, atol=2e-2)
    assert int(ops.tc_fault()[0]) == 0, "a wait inside the kernel ran out"
    # a row alone gives the same numbers as the row in the batch
    r = n // 2
    alone = ops.gemm_swap(a[r:r + 1].cuda(), w.cuda())
    assert torch.equal(alone[0], ops.gemm_swap(a.cuda(), w.cuda())[r])


@pytest.mark.parametrize("n", [1, 8, 40, 64])
@pytest.mark.parametrize("K,F", [(1536, 4096), (120, 352), (64, 32)])
def test_tcgen05_gemm_with_swapped_operands_and_swiglu_epilogue(n, K, F):
    ops = _ops()
    g = torch.Generator().manual_seed(62)
    a = _rand((n, K), torch.bfloat16, g)
    w = _rand((K, 2 * F), torch.bfloat16, g, 0.05)
    gu = (a.double() @ w.double()).reshape(n, F // 32, 2, 32)
    want = (torch.nn.functional.silu(gu[:, :, 0]) * gu[:, :, 1]).reshape(n, F)
    got = ops.gemm_swap(a.cuda(), w.cuda(), swiglu=True)
    assert got.shape == (n, F)
    torch.testing.assert_close(got.cpu().double(), want, rtol=2e-2, atol=2e-2)
    assert int(ops.tc_fault()[0]) == 0


@pytest.mark.parametrize("kernel", ["boxes", "ring"])
@pytest.mark.parametrize("n", [1, 8, 40, 64])
@pytest.mark.parametrize("K,F", [(1536, 4096), (120, 352), (64, 32)])
def test_skinny_gemm_with_swiglu_epilogue(n, K, F, kernel, monkeypatch):
    ops = _ops()
    monkeypatch.setattr(ops, "STREAM_GEMM", kernel != "ring")
    monkeypatch.setattr(ops, "STREAM_MIN_KC", 0)
    monkeypatch.setattr(ops, "STREAM_MAX_KC", 1 << 30)
    monkeypatch.setattr(ops, "STREAM_MAX_CTAS", 1 << 30)
    monkeypatch.setattr(ops, "STREAM_MAX_ROWS", 64)
    monkeypatch.setattr(ops, "SKINNY_SWIGLU_MAX_ROWS", 64)
    g = torch.Generator().manual_seed(13)
    a = _rand((n, K), torch.bfloat16, g)
    w = _rand((K, 2 * F), torch.bfloat16, g, 0.05)
    gu = (a.double() @ w.double()).reshape(n, F // 32, 2, 32)
    want = (torch.nn.functional.silu(gu[:, :, 0]) * gu[:, :, 1]).reshape(n, F)
    got = ops.gemm_swiglu(a.cuda(), w.cuda(), F, 32)
    assert got.shape == (n, F)
    torch.testing.assert_close(got.cpu().double(), want, rtol=2e-2, atol=2e-2)
    # more rows than the kernel takes: the library product and the gating kernel, same result
    if n == 64:
        a2 = _rand((80, K), torch.bfloat16, g)
        gu2 = (a2.double() @ w.double()).reshape(80, F // 32, 2, 32)
        want2 = (torch.nn.functional.silu(gu2[:, :, 0]) * gu2[:, :, 1]).reshape(80, F)
        torch.testing.assert_close(ops.gemm_swiglu(a2.cuda(), w.cuda(), F, 32).cpu().double(), want2, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("kernel", ["boxes", "ring", "swapped"])
@pytest.mark.parametrize("n", [1, 5, 8, 16, 33, 64])
@pytest.mark.parametrize("K,N", [(1536, 1536), (4096, 1536), (200, 120), (72, 8), (1000, 1096)])
def test_skinny_gemm_adds_to_the_stream_and_defers_the_norm(n, K, N, kernel, monkeypatch):
    """The residual epilogue (stream += product; stream * next norm's weight; partial sums of squares) and the
    product that applies the norm's factor per row afterwards, together against add + norm + product in float64.
    eps is large, so a factor with eps in the wrong place would show."""
    ops = _ops()
    monkeypatch.setattr(ops, "STREAM_GEMM", kernel != "ring")
    monkeypatch.setattr(ops, "STREAM_MIN_KC", 0)
    monkeypatch.setattr(ops, "STREAM_MAX_KC", 1 << 30)
    monkeypatch.setattr(ops, "STREAM_MAX_CTAS", 1 << 30)
    monkeypatch.setattr(ops, "STREAM_MAX_ROWS", 64)
    monkeypatch.setattr(ops, "SKINNY_MAX_ROWS", 64)
    monkeypatch.setattr(ops, "SKINNY_SWIGLU_MAX_ROWS", 64)
    g = torch.Generator().manual_seed(21)
    a = _rand((n, K), torch.bfloat16, g)
    w = _rand((K, N), torch.bfloat16, g, 0.05)
    stream = _rand((n, N), torch.float32, g, 2.0)
    stream[0] *= 30.0                                        # rows of very different length
    weight = 1.0 + _rand((N,), torch.float32, g, 0.3)
    eps = 0.75
    new_stream = stream.double() + a.double() @ w.double()
    normed = new_stream * math.sqrt(N) / (new_stream.norm(dim=-1, keepdim=True) + eps) * weight.double()
    F = 64
    w2 = _rand((N, 2 * F), torch.bfloat16, g, 0.05)
    want2 = normed @ w2.double()
    factor = math.sqrt(N) / (new_stream.norm(dim=-1, keepdim=True) + eps)
    swapped = kernel == "swapped"               # the tcgen05 kernel with swapped operands has the same epilogues
    product = ops.gemm_swap if swapped else ops.gemm_skinny
    for ksplit in (None, 1, 2, 4, 8):
        values = stream.cuda()
        sink = ops.ResidualSink(values, weight.cuda(), eps, norm="the norm")
        rows = product(a.cuda(), w.cuda(), ksplit=ksplit, sink=sink)
        assert isinstance(rows, ops.ScaledRows) and rows.norm == "the norm" and rows.parts.shape == (n, -(-N // 64))
        torch.testing.assert_close(values.cpu().double(), new_stream, rtol=1e-3, atol=2e-2)
        torch.testing.assert_close(rows.rows.cpu().double(), new_stream * weight.double(), rtol=1e-2, atol=2e-2)
        pad = torch.zeros(n, -(-N // 64) * 64, dtype=torch.float64)
        pad[:, :N] = values.cpu().double() ** 2
        torch.testing.assert_close(rows.parts.cpu().double(), pad.reshape(n, -1, 64).sum(-1), rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(rows.dense().cpu().double(), normed, rtol=2e-2, atol=2e-2)
        got2 = ops.gemm_swap(rows, w2.cuda(), ksplit=ksplit) if swapped else ops.gemm(rows, w2.cuda())
        torch.testing.assert_close(got2.cpu().double(), want2, rtol=2e-2, atol=2e-2)
        # the gated product against the same product of the rows as they were rounded to bfloat16
        gu = ((rows.rows.cpu().double() * factor) @ w2.double()).reshape(n, F // 32, 2, 32)
        want_gated = (torch.nn.functional.silu(gu[:, :, 0]) * gu[:, :, 1]).reshape(n, F)
        gated = ops.gemm_swap(rows, w2.cuda(), swiglu=True, ksplit=ksplit) if swapped else ops.gemm_swiglu(rows, w2.cuda(), F, 32)
        torch.testing.assert_close(gated.cpu().double(), want_gated, rtol=2e-2, atol=2e-2)
    # the same through the norm kernel: both ways agree to rounding
    values = stream.cuda()
    delta = ops.gemm_skinny(a.cuda(), w.cuda())
    x = ops.add_rmsnorm(values, delta, weight.cuda(), eps, torch.empty((n, N), dtype=torch.bfloat16, device="cuda"))
    torch.testing.assert_close(ops.gemm(x, w2.cuda()).cpu().double(), got2.cpu().double(), rtol=2e-2, atol=2e-2)
    if ops._tc_fault is not None:
        assert int(ops._tc_fault[0]) == 0, "a wait inside the kernel ran out"


@pytest.mark.parametrize("kernel", ["ring", "boxes", "swapped"])
def test_the_other_norm_factor(kernel, monkeypatch):
    """Rows whose norm is rsqrt(mean of squares + eps) (the "mean_eps" factor) instead of this architecture's
    sqrt(d) / (norm + eps): the products apply that factor from the same partial sums, and so does ``dense()``."""
    ops = _ops()
    monkeypatch.setattr(ops, "STREAM_GEMM", kernel == "boxes")
    monkeypatch.setattr(ops, "STREAM_MIN_KC", 0)
    monkeypatch.setattr(ops, "STREAM_MAX_KC", 1 << 30)
    g = torch.Generator().manual_seed(23)
    n, K, N, eps = 6, 328, 136, 0.3
    stream = _rand((n, K), torch.float32, g, 1.5)
    stream[1] *= 0.01                                            # a row for which eps decides
    weight = 1.0 + _rand((K,), torch.float32, g, 0.3)
    operand = (stream * weight).to(torch.bfloat16)
    parts = torch.nn.functional.pad(stream.pow(2), (0, -K % 64)).reshape(n, -1, 64).sum(-1)
    rows = ops.ScaledRows(operand.cuda(), parts.cuda(), eps, kind="mean_eps")
    factor = 1.0 / torch.sqrt(stream.double().pow(2).mean(-1, keepdim=True) + eps)
    other = math.sqrt(K) / (stream.double().norm(dim=-1, keepdim=True) + eps)
    assert ((factor - other).abs() / factor).max() > 0.2        # the two factors differ where eps matters
    w = _rand((K, N), torch.bfloat16, g, 0.05)
    want = (operand.double() * factor) @ w.double()
    got = (ops.gemm_swap if kernel == "swapped" else ops.gemm_skinny)(rows, w.cuda())
    torch.testing.assert_close(got.cpu().double(), want, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(rows.dense().cpu().double(), operand.double() * factor, rtol=1e-2, atol=1e-2)
    with pytest.raises(ops.KernelError):
        ops.ResidualSink(torch.zeros(1, 8), torch.ones(8), 0.0, kind="layer_norm")


def test_a_sink_is_ignored_by_products_that_cannot_use_it(monkeypatch):
    """More rows than the weight-streaming kernels take, or float32: the product returns its result and leaves
    the stream alone; rows whose factor is pending are made whole for a product that cannot apply it."""
    ops = _ops()
    g = torch.Generator().manual_seed(22)
    K, N = 256, 128
    w = _rand((K, N), torch.bfloat16, g, 0.05).cuda()
    weight = torch.ones(N, device="cuda")
    a = _rand((ops.SKINNY_MAX_ROWS + 9, K), torch.bfloat16, g).cuda()
    values = torch.zeros((a.shape[0], N), device="cuda")
    assert not ops.sink_usable(values, torch.bfloat16)
    got = ops.gemm(a, w, sink=ops.ResidualSink(values, weight, 1e-6))
    assert isinstance(got, torch.Tensor) and float(values.abs().max()) == 0.0
    torch.testing.assert_close(got.cpu().double(), a.cpu().double() @ w.cpu().double(), rtol=2e-2, atol=2e-2)
    few = a[:3].contiguous()
    small = torch.zeros((3, N), device="cuda")
    assert ops.sink_usable(small, torch.bfloat16) and not ops.sink_usable(small, torch.float32)
    rows = ops.gemm(few, w, sink=ops.ResidualSink(small, weight, 1e-6))
    assert isinstance(rows, ops.ScaledRows)
    monkeypatch.setattr(ops, "SKINNY_MAX_ROWS", 0)           # now every product is the library's
    monkeypatch.setattr(ops, "STREAM_GEMM", False)
    w2 = _rand((N, 72), torch.bfloat16, g, 0.05).cuda()
    got = ops.gemm(rows, w2)
    want = small.cpu().double()
    want = want * math.sqrt(N) / (want.norm(dim=-1, keepdim=True) + 1e-6)
    torch.testing.assert_close(got.cpu().double(), want @ w2.cpu().double(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("M,K,N", [(128, 64, 128), (300, 72, 200), (1000, 264, 1544), (2048, 1536, 2304),
                                   (513, 4096, 1536), (129, 40, 8), (640, 128, 448)])
def test_tcgen05_gemm(M, K, N):
    """The tcgen05 product for many rows: every tile width, rows, columns and K that do not fill
    their tiles, operands and results that are slices of wider matrices."""
    ops = _ops()
    g = torch.Generator().manual_seed(14)
    a = _rand((M, K), torch.bfloat16, g)
    w = _rand((K, N), torch.bfloat16, g, 0.05)
    want = a.double() @ w.double()
    tol = dict(rtol=2e-2, atol=2e-2 * max(1.0, float(want.abs().max()) / 4))
    got = ops.gemm_tc(a.cuda(), w.cuda())
    assert got.shape == (M, N) and got.dtype == torch.bfloat16
    torch.testing.assert_close(got.cpu().double(), want, **tol)
    wide_a = torch.zeros(M, K + 24, dtype=torch.bfloat16).cuda()
    wide_a[:, 8:8 + K] = a.cuda()
    wide_w = _rand((K, N + 64), torch.bfloat16, g, 0.05).cuda()
    wide_w[:, 16:16 + N] = w.cuda()
    out = torch.full((M, N + 16), 7.0, dtype=torch.bfloat16).cuda()
    ops.gemm_tc(wide_a[:, 8:8 + K], wide_w[:, 16:16 + N], out=out[:, 8:8 + N])
    torch.testing.assert_close(out[:, 8:8 + N].cpu().double(), want, **tol)
    assert bool((out[:, :8] == 7).all()) and bool((out[:, 8 + N:] == 7).all()), "wrote outside its columns"
    assert int(ops.tc_fault()[0]) == 0


@pytest.mark.parametrize("M,K,F", [(128, 64, 32), (130, 40, 96), (2048, 1536, 4096), (700, 200, 352)])
def test_tcgen05_gemm_with_swiglu_epilogue(M, K, F):
    ops = _ops()
    g = torch.Generator().manual_seed(15)
    a = _rand((M, K), torch.bfloat16, g)
    w = _rand((K, 2 * F), torch.bfloat16, g, 0.05)
    gu = (a.double() @ w.double()).reshape(M, F // 32, 2, 32)
    want = (torch.nn.functional.silu(gu[:, :, 0]) * gu[:, :, 1]).reshape(M, F)
    got = ops.gemm_tc(a.cuda(), w.cuda(), swiglu=True)
    assert got.shape == (M, F)
    torch.testing.assert_close(got.cpu().double(), want, rtol=2e-2, atol=2e-2 * max(1.0, float(want.abs().max()) / 4))
    assert int(ops.tc_fault()[0]) == 0


def test_tcgen05_gemm_refuses_what_tma_cannot_address():
    ops = _ops()
    a = torch.zeros(128, 36, dtype=torch.bfloat16).cuda()          # K not a multiple of 8
    w = torch.zeros(36, 64, dtype=torch.bfloat16).cuda()
    with pytest.raises(ops.KernelError, match="multiples of 8"):
        ops.gemm_tc(a, w)
    a = torch.zeros(128, 64, dtype=torch.bfloat16).cuda()
    w = torch.zeros(64, 96, dtype=torch.bfloat16).cuda()           # gated columns come in blocks of 64
    with pytest.raises(ops.KernelError, match="multiple of 64"):
        ops.gemm_tc(a, w, swiglu=True)


@pytest.mark.parametrize("dtype", DTYPES)
def test_residual_add(dtype):
    ops = _ops()
    g = torch.Generator().manual_seed(3)
    res = torch.randn(9, 130, generator=g)
    delta = _rand((9, 130), dtype, g)
    want = res + delta.float()
    got = ops.residual_add(res.cuda(), delta.cuda())
    torch.testing.assert_close(got.cpu(), want, rtol=1e-6, atol=1e-6)


def _scattered_tables(n_slots, max_pages, num_pages, gen):
    perm = torch.randperm(num_pages, generator=gen)
    table = torch.full((n_slots, max_pages), -1, dtype=torch.int32)
    k = 0
    for s in range(n_slots):
        for p in range(max_pages):
            if k < num_pages:
                table[s, p] = perm[k]
                k += 1
    return table


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,KVH,hd,page,rot,inter", [(4, 2, 16, 16, None, False), (6, 2, 48, 4, None, False),
                                                      (5, 5, 32, 8, 16, False), (3, 1, 64, 32, None, True),
                                                      (12, 3, 128, 16, None, False)])
def test_rope_kv_write(dtype, H, KVH, hd, page, rot, inter):
    ops = _ops()
    g = torch.Generator().manual_seed(4)
    n, slots, max_pages = 11, 3, 6
    num_pages = slots * max_pages
    rot = rot or hd
    table = _scattered_tables(slots, max_pages, num_pages, g)
    qkv = _rand((n, (H + 2 * KVH) * hd), dtype, g)
    positions = torch.tensor([0, 1, 2, 3, page - 1, page, page * 2 - 1, page * 2, 5, 0, 9], dtype=torch.int32)
    row_slot = torch.tensor([0, 0, 0, 0, 1, 1, 1, 1, 2, -1, 2], dtype=torch.int32)
    ang = torch.outer(torch.arange(80, dtype=torch.float64), 10000.0 ** (-2.0 * torch.arange(rot // 2) / rot))
    cos, sin = torch.cos(ang).float(), torch.sin(ang).float()
    plane = torch.zeros(num_pages, 2, KVH, page, hd, dtype=dtype)
    fault = torch.zeros(4, dtype=torch.int32)
    qkv_ref, plane_ref = qkv.clone(), plane.clone()
    ref.rope_kv_write(qkv_ref, positions, row_slot, cos, sin, plane_ref, table, H, KVH, hd, page, fault,
                      interleaved=inter)
    qkv_dev, plane_dev, fault_dev = qkv.cuda(), plane.cuda(), fault.cuda()
    ops.rope_kv_write(qkv_dev, positions.cuda(), row_slot.cuda(), cos.cuda(), sin.cuda(), plane_dev, table.cuda(),
                      H, KVH, hd, page, fault_dev, interleaved=inter)
    tol = dict(rtol=1e-6, atol=1e-6) if dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2)
    valid = row_slot >= 0
    torch.testing.assert_close(qkv_dev.cpu()[valid].float(), qkv_ref[valid].float(), **tol)
    torch.testing.assert_close(plane_dev.cpu().float(), plane_ref.float(), **tol)
    assert int(fault_dev[0]) == 0
    # the padding row wrote nothing and was not rotated
    assert torch.equal(qkv_dev.cpu()[9], qkv[9])

    # many rows (a warp per row): 70 rows of one request at positions 3..72, a padding row in the middle
    n2 = 71
    table2 = _scattered_tables(1, 80 // page + 1, 80 // page + 4, g)
    qkv2 = _rand((n2, (H + 2 * KVH) * hd), dtype, g)
    pos2 = torch.tensor(list(range(3, 40)) + [0] + list(range(40, 73)), dtype=torch.int32)
    slot2 = torch.tensor([0] * 37 + [-1] + [0] * 33, dtype=torch.int32)
    plane2 = torch.zeros(80 // page + 4, 2, KVH, page, hd, dtype=dtype)
    q_ref, p_ref = qkv2.clone(), plane2.clone()
    ref.rope_kv_write(q_ref, pos2, slot2, cos, sin, p_ref, table2, H, KVH, hd, page, fault, interleaved=inter)
    q_dev, p_dev = qkv2.cuda(), plane2.cuda()
    ops.rope_kv_write(q_dev, pos2.cuda(), slot2.cuda(), cos.cuda(), sin.cuda(), p_dev, table2.cuda(), H, KVH, hd, page,
                      fault_dev, interleaved=inter)
    ok = slot2 >= 0
    torch.testing.assert_close(q_dev.cpu()[ok].float(), q_ref[ok].float(), **tol)
    torch.testing.assert_close(p_dev.cpu().float(), p_ref.float(), **tol)
    assert torch.equal(q_dev.cpu()[37], qkv2[37]) and int(fault_dev[0]) == 0


def test_rope_kv_write_reports_bad_page():
    ops = _ops()
    H, KVH, hd, page = 2, 1, 16, 4
    qkv = torch.randn(1, (H + 2 * KVH) * hd).cuda()
    table = torch.tensor([[99]], dtype=torch.int32).cuda()          # outside a pool of 2 pages
    plane = torch.zeros(2, 2, KVH, page, hd).cuda()
    fault = torch.zeros(4, dtype=torch.int32).cuda()
    cos = torch.ones(8, hd // 2).cuda()
    sin = torch.zeros(8, hd // 2).cuda()
    ops.rope_kv_write(qkv, torch.zeros(1, dtype=torch.int32).cuda(), torch.zeros(1, dtype=torch.int32).cuda(),
                      cos, sin, plane, table, H, KVH, hd, page, fault)
    assert int(fault[0]) != 0
    assert float(plane.abs().sum()) == 0.0


def _fill_cache(dtype, slots_len, KVH, hd, page, gen, scale=1.0):
    """Random keys and values for each slot, written into scattered pages."""
    max_pages = max((L + page - 1) // page for L in slots_len) + 1
    num_pages = len(slots_len) * max_pages + 3
    table = _scattered_tables(len(slots_len), max_pages, num_pages, gen)
    plane = torch.zeros(num_pages, 2, KVH, page, hd, dtype=dtype)
    for s, L in enumerate(slots_len):
        k = _rand((L, KVH, hd), dtype, gen, scale)
        v = _rand((L, KVH, hd), dtype, gen)
        for t in range(L):
            pg = int(table[s, t // page])
            plane[pg, 0, :, t % page] = ref.cache_row(k[t], t)
            plane[pg, 1, :, t % page] = ref.cache_row(v[t], t)
    return plane, table


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,KVH,hd,page,window", [(4, 2, 16, 16, None), (6, 2, 48, 4, None), (8, 2, 64, 16, None),
                                                  (5, 5, 32, 8, 20), (12, 3, 128, 16, None), (3, 1, 80, 32, 37),
                                                  (7, 7, 256, 16, None), (16, 1, 112, 8, None)])
def test_paged_attention(dtype, H, KVH, hd, page, window):
    ops = _ops()
    g = torch.Generator().manual_seed(5)
    lens = [37, 300, 1, 130]
    plane, table = _fill_cache(dtype, lens, KVH, hd, page, g)
    # rows: decode rows at the end of each slot, a chunk of rows inside slot 1, a padding row
    rows = [(0, 36), (1, 299), (2, 0), (3, 129)] + [(1, p) for p in range(120, 140)] + [(-1, 0), (3, 64), (3, 15),
                                                                                         (3, 16), (0, 0)]
    row_slot = torch.tensor([r[0] for r in rows], dtype=torch.int32)
    positions = torch.tensor([r[1] for r in rows], dtype=torch.int32)
    n = len(rows)
    stride = (H + 2 * KVH) * hd
    q = _rand((n, stride), dtype, g)
    fault = torch.zeros(4, dtype=torch.int32)
    want = ref.paged_attention(q, torch.empty(n, H * hd, dtype=dtype), plane, table, positions, row_slot, H, KVH, hd,
                               page, window, fault)
    fault_dev = fault.cuda()
    got = ops.paged_attention(q.cuda(), torch.empty(n, H * hd, dtype=dtype, device="cuda"), plane.cuda(),
                              table.cuda(), positions.cuda(), row_slot.cuda(), H, KVH, hd, page, window, fault_dev)
    tol = dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(got.cpu().float(), want.float(), **tol)
    assert int(fault_dev[0]) == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_paged_attention_finds_a_far_key(dtype):
    """One key among hundreds, at a page's first slot far back, is made to stand out: its
    value must dominate the output.  A kernel that skips a page, or reads a neighbour's,
    fails here although random inputs would hide it."""
    ops = _ops()
    g = torch.Generator().manual_seed(6)
    H, KVH, hd, page = 4, 2, 32, 16
    L = 700
    plane, table = _fill_cache(dtype, [L], KVH, hd, page, g, scale=0.1)
    n = 3
    q = _rand((n, (H + 2 * KVH) * hd), dtype, g, 0.1)
    for far in (0, 16 * 7, 16 * 30 + 15):
        pl = plane.clone()
        pg = int(table[0, far // page])
        marker = torch.zeros(hd)
        marker[3] = 30.0
        pl[pg, 0, :, far % page] = ref.cache_row(marker.to(dtype), far)   # key: large along one axis
        pl[pg, 1, :, far % page] = torch.full((hd,), 5.0).to(dtype)       # value: easy to recognise
        qq = q.clone()
        qq[:, : H * hd] = 0
        for h in range(H):
            qq[:, h * hd + 3] = 30.0                         # every query looks along that axis
        positions = torch.tensor([L - 1, L - 2, far], dtype=torch.int32)
        row_slot = torch.zeros(n, dtype=torch.int32)
        fault = torch.zeros(4, dtype=torch.int32).cuda()
        got = ops.paged_attention(qq.cuda(), torch.empty(n, H * hd, dtype=dtype, device="cuda"), pl.cuda(),
                                  table.cuda(), positions.cuda(), row_slot.cuda(), H, KVH, hd, page, None, fault)
        assert (got.float() - 5.0).abs().max() < 0.05, f"far key at {far} not found"
        want = ref.paged_attention(qq, torch.empty(n, H * hd, dtype=dtype), pl, table, positions, row_slot, H, KVH,
                                   hd, page, None, torch.zeros(4, dtype=torch.int32))
        torch.testing.assert_close(got.cpu().float(), want.float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_paged_attention_window_edge(dtype):
    """The key just outside the window is made to stand out and must be ignored; the key
    just inside must be seen."""
    ops = _ops()
    g = torch.Generator().manual_seed(7)
    H, KVH, hd, page, W = 2, 1, 16, 8, 24
    L = 100
    base, table = _fill_cache(dtype, [L], KVH, hd, page, g, scale=0.05)
    pos = 90
    for key_pos, seen in ((pos - W, False), (pos - W + 1, True)):
        pl = base.clone()
        pg = int(table[0, key_pos // page])
        marker = torch.zeros(hd)
        marker[0] = 40.0
        pl[pg, 0, 0, key_pos % page] = ref.cache_row(marker.to(dtype), key_pos)
        pl[pg, 1, 0, key_pos % page] = torch.full((hd,), 9.0).to(dtype)
        q = torch.zeros(1, (H + 2 * KVH) * hd)
        q[0, 0] = 40.0
        q[0, hd] = 40.0
        q = q.to(dtype)
        fault = torch.zeros(4, dtype=torch.int32).cuda()
        got = ops.paged_attention(q.cuda(), torch.empty(1, H * hd, dtype=dtype, device="cuda"), pl.cuda(),
                                  table.cuda(), torch.tensor([pos], dtype=torch.int32).cuda(),
                                  torch.zeros(1, dtype=torch.int32).cuda(), H, KVH, hd, page, W, fault)
        if seen:
            assert (got.float() - 9.0).abs().max() < 0.1
        else:
            assert got.float().abs().max() < 1.0


@pytest.mark.parametrize("path,start,n", [("rows", 300, 160), ("groups3", 0, 700), ("tc", 300, 160), ("tc", 0, 700)])
@pytest.mark.parametrize("H,KVH,hd,page,W", [(8, 2, 128, 16, 128), (4, 2, 64, 32, 64), (6, 2, 128, 64, 192)])
def test_window_edge_in_prompt_portions(path, start, n, H, KVH, hd, page, W, monkeypatch):
    """The edge of the window for rows inside tiles of many rows (the row-tile kernel, its variant with three
    key groups, the tcgen05 kernel): for chosen rows — the first, a middle and the last row of a tile, on both
    sides of tile borders — the key just inside the window is made to stand out for that row alone, and the key
    just outside to stand out more still.  A row that sees one key too many, or one too few, comes out as
    another value row altogether.  The window is a multiple of the page and of the 64-key tile, so
    the edges of the chosen rows fall on page and tile borders as well as inside them; two padding rows of a
    stage that runs behind lead the portion."""
    from tiny_inference_server_b200.kernels.attention_plan import TileSet, plan_tiles
    ops = _ops()
    g = torch.Generator().manual_seed(51)
    dtype = torch.bfloat16
    L = start + n
    plane, table = _fill_cache(dtype, [L], KVH, hd, page, g)
    pad = 2
    chosen = sorted({r for r in (0, 15, 16, 40, 63, 64, 100, 127, 128, 159, 200, 255, 256, 511, 512, n - 1)
                     if r < n and start + r - W >= 0})
    assert len(chosen) >= 5

    # every chosen row looks along a direction of its own; its two keys point that way
    marks = {}
    for i, r in enumerate(chosen):
        d = 3 + 2 * i
        marks.setdefault(start + r - W, torch.zeros(hd))[d] = 120.0        # just outside the window of row r
        marks.setdefault(start + r - W + 1, torch.zeros(hd))[d] = 80.0     # just inside
    for pos, m in marks.items():
        pg = int(table[0, pos // page])
        for kvh in range(KVH):
            plane[pg, 0, kvh, pos % page] = ref.cache_row(m.to(dtype), pos)
    rows = [(-1, 0)] * pad + [(0, start + r) for r in range(n)]
    row_slot = torch.tensor([r[0] for r in rows], dtype=torch.int32)
    positions = torch.tensor([r[1] for r in rows], dtype=torch.int32)
    q = _rand((n + pad, (H + 2 * KVH) * hd), dtype, g, 0.3)
    for i, r in enumerate(chosen):
        for h in range(H):
            q[pad + r, h * hd: (h + 1) * hd] = 0.0
            q[pad + r, h * hd + 3 + 2 * i] = 8.0
    fault = torch.zeros(4, dtype=torch.int32)
    want = ref.paged_attention(q, torch.empty(n + pad, H * hd, dtype=dtype), plane, table, positions, row_slot, H, KVH,
                               hd, page, W, fault)
    # the tiles as the engine makes them: the padding rows belong to the segment that follows them
    keys, rws, wide, rows_in_wide = plan_tiles([(0, n + pad)], H // KVH)

    def t(v):
        return torch.tensor(v, dtype=torch.int32, device="cuda")

    tiles = TileSet((t([k[0] for k in keys]), t([k[1] for k in keys]), len(keys)),
                    (t([k[0] for k in rws]), t([k[1] for k in rws]), len(rws)), max((k[1] for k in keys), default=0),
                    (t([k[0] for k in wide]), t([k[1] for k in wide]), len(wide)), rows_in_wide)

    class Step:
        decode_only = False
        max_position, min_position = L - 1, start

        def plan(self, planner):
            return tiles

    monkeypatch.setattr(ops, "TC_ATTENTION", path == "tc")
    monkeypatch.setattr(ops, "TC_ATTENTION_MIN_TILES", 1)
    before = dict(ops.calls)
    fault_dev = fault.cuda()
    got = ops.paged_attention(q.cuda(), torch.full((n + pad, H * hd), 7.0, dtype=dtype, device="cuda"), plane.cuda(),
                              table.cuda(), positions.cuda(), row_slot.cuda(), H, KVH, hd, page, W, fault_dev, Step())
    torch.cuda.synchronize()
    assert int(fault_dev[0]) == 0
    assert (ops.calls["attn_tc"] - before.get("attn_tc", 0) == 1) == (path == "tc")
    if path != "tc":
        assert ops.calls["attn_rows"] - before.get("attn_rows", 0) == 1
    got = got.cpu().float()
    valid = row_slot >= 0
    torch.testing.assert_close(got[valid], want.float()[valid], rtol=2e-2, atol=2e-2)
    for r in chosen:                       # the key just inside wins: its value row comes out, for every head
        pos = start + r - W + 1
        pg = int(table[0, pos // page])
        for h in range(H):
            v = ref.cache_row_inverse(plane[pg, 1, h // (H // KVH), pos % page], pos).float()
            torch.testing.assert_close(got[pad + r, h * hd:(h + 1) * hd], v, rtol=5e-2, atol=5e-2)


def test_paged_attention_refuses_bad_head_size():
    ops = _ops()
    from tiny_inference_server_b200.kernels.ops import KernelError
    z = torch.zeros(1, 3 * 24, device="cuda")
    with pytest.raises(KernelError):
        ops.paged_attention(z, torch.zeros(1, 24, device="cuda"), torch.zeros(1, 2, 1, 4, 24, device="cuda"),
                            torch.zeros(1, 1, dtype=torch.int32, device="cuda"),
                            torch.zeros(1, dtype=torch.int32, device="cuda"),
                            torch.zeros(1, dtype=torch.int32, device="cuda"), 1, 1, 24, 4, None,
                            torch.zeros(4, dtype=torch.int32, device="cuda"))


@pytest.mark.parametrize("dtype", DTYPES)
def test_mtp_input(dtype):
    ops = _ops()
    g = torch.Generator().manual_seed(8)
    n, d, V, slots = 9, 72, 50, 4
    h_prev = _rand((n, d), dtype, g)
    state = _rand((slots, d), dtype, g)
    row_slot = torch.tensor([2, 2, 2, 0, 3, 3, -1, 1, 1], dtype=torch.int32)
    row_last = torch.tensor([2, 2, 2, 3, 5, 5, 6, 8, 8], dtype=torch.int32)
    tokens = torch.randint(0, V, (n,), generator=g, dtype=torch.int32)
    table = _rand((V, d), dtype, g)
    scale = 1 + 0.1 * torch.randn(d, generator=g)
    state_ref = state.clone()
    want = ref.mtp_input(h_prev, state_ref, row_slot, row_last, tokens, table, scale, 1e-5,
                         torch.zeros(n, 2 * d, dtype=dtype))
    state_dev = state.cuda()
    got = ops.mtp_input(h_prev.cuda(), state_dev, row_slot.cuda(), row_last.cuda(), tokens.cuda(), table.cuda(),
                        scale.cuda(), 1e-5, torch.zeros(n, 2 * d, dtype=dtype, device="cuda"))
    torch.testing.assert_close(got.cpu().float(), want.float(), **_tol(dtype))
    torch.testing.assert_close(state_dev.cpu().float(), state_ref.float(), rtol=0, atol=0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,K,N", [(1, 64, 48), (7, 120, 301), (64, 1536, 2304), (130, 200, 120)])
def test_gemm(dtype, n, K, N):
    ops = _ops()
    g = torch.Generator().manual_seed(9)
    a = _rand((n, K), dtype, g)
    w = _rand((K, N), dtype, g, 0.05)
    want = a.double() @ w.double()
    got = ops.gemm(a.cuda(), w.cuda())
    assert got.dtype == dtype
    tol = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(got.cpu().double(), want, **tol)
    got32 = ops.gemm_f32_out(a.cuda(), w.cuda())
    assert got32.dtype == torch.float32
    tol = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(got32.cpu().double(), want, **tol)


@pytest.mark.parametrize("n,K,N,kernel", [(5, 1536, 2304, "gemm_skinny"), (3, 4096, 4096, "gemm_skinny"),
                                          (8, 4096, 1536, "gemm_stream"), (5, 8192, 200, "gemm_swap"),
                                          (6, 14336, 4096, "gemm_swap"), (6, 3072, 5120, "gemm_library"),
                                          (9, 1536, 2304, "gemm_skinny"), (33, 1536, 2304, "gemm_library")])
def test_few_rows_go_to_the_kernel_their_shape_calls_for(n, K, N, kernel):
    """Few bfloat16 rows: a short share of K per CTA goes to the ring (or, one round of boxes, to the TMA-fed kernel),
    a long share to the tcgen05 kernel with swapped operands when the matrix is tall, else to the library; with a
    sink and rows whose norm factor is pending, every one of them gives the same result as add + norm + product."""
    ops = _ops()
    g = torch.Generator().manual_seed(19)
    a = _rand((n, K), torch.bfloat16, g)
    w = _rand((K, N), torch.bfloat16, g, 0.03).cuda()
    before = dict(ops.calls)
    got = ops.gemm(a.cuda(), w)
    ran = {k for k, v in ops.calls.items() if v != before.get(k, 0)}
    assert ran == {kernel}, ran
    torch.testing.assert_close(got.cpu().double(), a.double() @ w.cpu().double(), rtol=2e-2, atol=2e-2)
    # the same product fed with rows whose factor is pending and told to add to a stream
    stream = _rand((n, K), torch.float32, g, 2.0)
    rows = ops.ScaledRows((stream * 1.5).to(torch.bfloat16).cuda(),
                          torch.nn.functional.pad(stream.pow(2), (0, -K % 64)).reshape(n, -1, 64).sum(-1).cuda(), 0.5)
    x = (stream * 1.5).to(torch.bfloat16).double() * math.sqrt(K) / (stream.double().norm(dim=-1, keepdim=True) + 0.5)
    target = _rand((n, N), torch.float32, g, 2.0)
    values = target.cuda()
    weight = (1.0 + _rand((N,), torch.float32, g, 0.3)).cuda()
    out = ops.gemm(rows, w, sink=ops.ResidualSink(values, weight, 0.25) if ops.sink_usable(values, torch.bfloat16) else None)
    want = x @ w.cpu().double()
    if isinstance(out, ops.ScaledRows):
        assert kernel != "gemm_library"
        torch.testing.assert_close(values.cpu().double(), target.double() + want, rtol=2e-2, atol=3e-2)
        torch.testing.assert_close(out.dense().cpu().double(),
                                   (values.cpu().double() * math.sqrt(N) / (values.cpu().double().norm(dim=-1, keepdim=True) + 0.25)
                                    * weight.cpu().double()), rtol=2e-2, atol=2e-2)
    else:
        assert kernel == "gemm_library"
        torch.testing.assert_close(out.cpu().double(), want, rtol=2e-2, atol=3e-2)
        assert torch.equal(values.cpu(), target)
    assert int(ops.tc_fault()[0]) == 0


def test_float32_products_are_not_tf32():
    """A product whose exact value needs more than TF32's 10 mantissa bits."""
    ops = _ops()
    a = torch.full((4, 256), 1.0 + 2.0 ** -12).cuda()
    w = torch.full((256, 8), 1.0).cuda()
    got = ops.gemm(a, w).cpu()
    assert abs(float(got[0, 0]) - 256 * (1.0 + 2.0 ** -12)) < 1e-4


@pytest.mark.parametrize("H,KVH,hd,page,window", [(12, 3, 128, 16, None), (4, 2, 16, 16, None), (6, 2, 48, 4, 50),
                                                  (8, 1, 64, 8, None), (5, 5, 32, 8, None), (32, 1, 80, 32, None),
                                                  (20, 1, 96, 16, 300), (2, 2, 256, 16, None)])
def test_paged_attention_tensor_core_long_context_and_portions(H, KVH, hd, page, window):
    """The bfloat16 kernels with key splits: decode rows over thousands of keys, portions of
    17 and 100 rows deep inside a context, every group size up to 32 (more than 16 query
    heads per kv head go through the row tiles)."""
    ops = _ops()
    g = torch.Generator().manual_seed(11)
    dtype = torch.bfloat16
    lens = [3000, 700, 64, 1]
    plane, table = _fill_cache(dtype, lens, KVH, hd, page, g)
    rows = [(0, 2999), (1, 699), (2, 63), (3, 0)]
    rows += [(0, p) for p in range(1500, 1517)]            # a portion of 17 rows
    rows += [(1, p) for p in range(520, 620)]              # a portion of 100 rows
    rows += [(-1, 0), (2, 0), (2, 1)]
    row_slot = torch.tensor([r[0] for r in rows], dtype=torch.int32)
    positions = torch.tensor([r[1] for r in rows], dtype=torch.int32)
    n = len(rows)
    q = _rand((n, (H + 2 * KVH) * hd), dtype, g)
    fault = torch.zeros(4, dtype=torch.int32)
    want = ref.paged_attention(q, torch.empty(n, H * hd, dtype=dtype), plane, table, positions, row_slot, H, KVH, hd,
                               page, window, fault)
    fault_dev = fault.cuda()
    got = ops.paged_attention(q.cuda(), torch.full((n, H * hd), 7.0, dtype=dtype, device="cuda"), plane.cuda(),
                              table.cuda(), positions.cuda(), row_slot.cuda(), H, KVH, hd, page, window, fault_dev)
    torch.testing.assert_close(got.cpu().float(), want.float(), rtol=2e-2, atol=2e-2)
    assert int(fault_dev[0]) == 0


@pytest.mark.parametrize("H,KVH,hd,page,window", [(12, 3, 128, 16, None), (8, 2, 64, 16, None), (4, 4, 32, 8, None),
                                                  (16, 1, 96, 32, None), (6, 2, 128, 64, 100), (32, 2, 64, 16, 40),
                                                  (3, 1, 256, 16, None)])
@pytest.mark.parametrize("write_kv", [True, False])
def test_decode_attention_with_rotary_and_cache_write_inside(H, KVH, hd, page, window, write_kv):
    """A decode step whose rotary encoding and cache write the attention kernel does itself, against the two
    launches it replaces (rope_kv_write, then attention): the same outputs bit for bit and the same pages.
    Contexts of one key, a page's edge, a tile's edge, thousands of keys (key splits), a padding row; with
    write_kv off (a layer that reads another layer's cache) the plane must stay untouched."""
    from tiny_inference_server_b200.kernels.attention_plan import infer_tiles
    ops = _ops()
    g = torch.Generator().manual_seed(41)
    dtype = torch.bfloat16
    lens = [1, page, page + 1, 64, 65, 700, 3000, 129]
    plane, table = _fill_cache(dtype, lens, KVH, hd, page, g)
    rows = [(s, L - 1) for s, L in enumerate(lens)]
    rows.insert(3, (-1, 0))                                   # a padding row of the bucket
    row_slot = torch.tensor([r[0] for r in rows], dtype=torch.int32)
    positions = torch.tensor([r[1] for r in rows], dtype=torch.int32)
    n = len(rows)
    qkv = _rand((n, (H + 2 * KVH) * hd), dtype, g)
    ang = torch.outer(torch.arange(3000, dtype=torch.float64),
                      torch.pow(torch.tensor(10000.0, dtype=torch.float64), -2.0 * torch.arange(hd // 2) / hd))
    cos, sin = torch.cos(ang).float().cuda(), torch.sin(ang).float().cuda()

    class Step:
        decode_only = True
        max_position, min_position = 2999, 0
        tiles = infer_tiles(positions.cuda(), row_slot.cuda(), H // KVH)

        def plan(self, planner):
            return self.tiles

    # the two launches
    fault = torch.zeros(4, dtype=torch.int32, device="cuda")
    q1, plane1 = qkv.cuda().clone(), plane.cuda().clone()
    ops.rope_kv_write(q1, positions.cuda(), row_slot.cuda(), cos, sin, plane1, table.cuda(), H, KVH, hd, page, fault,
                      write_kv=write_kv)
    want = ops.paged_attention(q1, torch.empty(n, H * hd, dtype=dtype, device="cuda"), plane1, table.cuda(),
                               positions.cuda(), row_slot.cuda(), H, KVH, hd, page, window, fault, Step())
    # one launch
    q2, plane2 = qkv.cuda().clone(), plane.cuda().clone()
    assert ops.rotary_fusable(q2, Step(), H, KVH, hd)
    before = ops.calls["attn_keys_rotary"]
    got = ops.paged_attention(q2, torch.full((n, H * hd), 7.0, dtype=dtype, device="cuda"), plane2, table.cuda(),
                              positions.cuda(), row_slot.cuda(), H, KVH, hd, page, window, fault, Step(),
                              rotary=(cos, sin), write_kv=write_kv)
    torch.cuda.synchronize()
    assert ops.calls["attn_keys_rotary"] == before + 1 and int(fault[0]) == 0
    assert torch.equal(q2, qkv.cuda()), "the projection's output is read only"
    valid = row_slot >= 0
    if write_kv:
        assert torch.equal(plane2, plane1), "the pages differ from what rope_kv_write leaves"
        assert torch.equal(got[valid.cuda()], want[valid.cuda()])
    else:
        assert torch.equal(plane2, plane.cuda()), "the plane was written with write_kv off"
        torch.testing.assert_close(got[valid.cuda()].float(), want[valid.cuda()].float(), rtol=0, atol=0)
    # and both equal the plain reference
    ref_q, ref_plane = qkv.clone(), plane.clone()
    ref.rope_kv_write(ref_q, positions, row_slot, cos.cpu(), sin.cpu(), ref_plane, table, H, KVH, hd, page,
                      torch.zeros(4, dtype=torch.int32), write_kv=write_kv)
    plain = ref.paged_attention(ref_q, torch.empty(n, H * hd, dtype=dtype), ref_plane, table, positions, row_slot, H,
                                KVH, hd, page, window, torch.zeros(4, dtype=torch.int32))
    torch.testing.assert_close(got.cpu().float()[valid], plain.float()[valid], rtol=2e-2, atol=2e-2)


def test_attention_splits_plan():
    from tiny_inference_server_b200.kernels.ops import plan_splits
    for tiles, kvh, max_kv, keys_mode in [(8, 3, 4096, True), (64, 3, 4096, True), (1, 1, 1, True), (1, 3, 100, True),
                                          (128, 3, 2048, False), (4, 3, 4096, False), (500, 8, 5000, True)]:
        per, splits = plan_splits(tiles, kvh, max_kv, keys_mode)
        assert per % 64 == 0 and per >= 64 and splits >= 1
        assert per * splits >= max_kv and per * (splits - 1) < max_kv
    # clusters of 16 only while the CTAs of the decode kernel are all resident (two to an SM)
    assert plan_splits(1, 3, 4096, True)[1] == 16 and plan_splits(4, 3, 4096, True)[1] == 16
    assert plan_splits(8, 3, 4096, True)[1] == 8 and plan_splits(64, 3, 4096, True)[1] <= 8


@pytest.mark.parametrize("H,KVH,hd,page,window", [(12, 3, 128, 16, None), (4, 4, 64, 8, None), (6, 2, 32, 16, None),
                                                  (8, 2, 128, 32, 200)])
def test_paged_attention_whole_long_prompt(H, KVH, hd, page, window):
    """A prompt of 700 tokens in one step: the row-tile kernel with three key groups per CTA
    (long prompts from their start), two requests side by side, one of them short."""
    from tiny_inference_server_b200.kernels.attention_plan import infer_tiles
    ops = _ops()
    g = torch.Generator().manual_seed(14)
    dtype = torch.bfloat16
    lens = [700, 90]
    plane, table = _fill_cache(dtype, lens, KVH, hd, page, g)
    rows = [(0, p) for p in range(700)] + [(1, p) for p in range(90)]
    row_slot = torch.tensor([r[0] for r in rows], dtype=torch.int32)
    positions = torch.tensor([r[1] for r in rows], dtype=torch.int32)
    n = len(rows)
    q = _rand((n, (H + 2 * KVH) * hd), dtype, g)
    fault = torch.zeros(4, dtype=torch.int32)
    want = ref.paged_attention(q, torch.empty(n, H * hd, dtype=dtype), plane, table, positions, row_slot, H, KVH, hd,
                               page, window, fault)

    class Step:                      # what the attention operation reads of a step
        max_position, min_position = 699, 0
        tiles = infer_tiles(positions.cuda(), row_slot.cuda(), H // KVH)

        def plan(self, planner):
            return self.tiles

    fault_dev = fault.cuda()
    got = ops.paged_attention(q.cuda(), torch.full((n, H * hd), 7.0, dtype=dtype, device="cuda"), plane.cuda(),
                              table.cuda(), positions.cuda(), row_slot.cuda(), H, KVH, hd, page, window, fault_dev, Step())
    torch.testing.assert_close(got.cpu().float(), want.float(), rtol=2e-2, atol=2e-2)
    assert int(fault_dev[0]) == 0


@pytest.mark.parametrize("H,KVH,hd,page,window", [(12, 3, 128, 16, None), (4, 1, 64, 16, None), (6, 2, 128, 64, None),
                                                  (2, 2, 64, 128, None), (8, 2, 128, 32, 150), (5, 5, 64, 16, 70)])
def test_tcgen05_attention(H, KVH, hd, page, window, monkeypatch):
    """The tcgen05 kernel for long portions (tiles of up to 128 rows): a prompt from its start,
    a portion deep inside a context, a tile of a single key tile, leading padding rows of a
    stage that runs behind (slot -1), and one key made to stand out far back; compared with the
    plain reference and with the mma.sync kernel on the same rows."""
    from tiny_inference_server_b200.kernels.attention_plan import infer_tiles, TileSet
    ops = _ops()
    g = torch.Generator().manual_seed(21)
    dtype = torch.bfloat16
    lens = [1400, 100, 300]
    plane, table = _fill_cache(dtype, lens, KVH, hd, page, g)
    # one key of slot 0 far back that every later row of head 0 must find: scale its key up
    far = 5 * page
    pg = int(table[0, far // page])
    marker = torch.zeros(hd)
    marker[3] = 40.0
    plane[pg, 0, 0, far % page] = ref.cache_row(marker.to(dtype), far)
    rows = [(0, p) for p in range(1000, 1300)]             # a portion of 300 rows deep inside: tiles 128+128+44
    rows += [(1, p) for p in range(100)]                   # a prompt from its start: one tile, one key tile
    rows += [(-1, 0), (-1, 0)] + [(2, p) for p in range(298)]   # a stage two positions behind: padding first
    row_slot = torch.tensor([r[0] for r in rows], dtype=torch.int32)
    positions = torch.tensor([r[1] for r in rows], dtype=torch.int32)
    n = len(rows)
    q = _rand((n, (H + 2 * KVH) * hd), dtype, g)
    q[:300, 3] = 8.0                                       # head 0 of the deep portion looks along the marker
    fault = torch.zeros(4, dtype=torch.int32)
    want = ref.paged_attention(q, torch.empty(n, H * hd, dtype=dtype), plane, table, positions, row_slot, H, KVH, hd,
                               page, window, fault)
    # the tiles as the engine makes them: the padding rows belong to the segment that follows them
    tiles = infer_tiles(positions.cuda(), row_slot.cuda(), H // KVH)
    segs = [(0, 300), (300, 100), (400, 300)]
    from tiny_inference_server_b200.kernels.attention_plan import plan_tiles
    keys, rws, wide, rows_in_wide = plan_tiles(segs, H // KVH)

    def t(v):
        return torch.tensor(v, dtype=torch.int32, device="cuda")

    tiles = TileSet((t([k[0] for k in keys]), t([k[1] for k in keys]), len(keys)),
                    (t([k[0] for k in rws]), t([k[1] for k in rws]), len(rws)), max((k[1] for k in keys), default=0),
                    (t([k[0] for k in wide]), t([k[1] for k in wide]), len(wide)), rows_in_wide)
    assert len(wide) == 7

    class Step:
        max_position, min_position = 1299, 0

        def plan(self, planner):
            return tiles

    monkeypatch.setattr(ops, "TC_ATTENTION_MIN_TILES", 1)     # also where the mma.sync kernel would be chosen
    outs = {}
    for tc in (True, False):
        ops.TC_ATTENTION = tc
        try:
            fault_dev = fault.cuda()
            tc_before = ops.calls["attn_tc"]
            got = ops.paged_attention(q.cuda(), torch.full((n, H * hd), 7.0, dtype=dtype, device="cuda"), plane.cuda(),
                                      table.cuda(), positions.cuda(), row_slot.cuda(), H, KVH, hd, page, window,
                                      fault_dev, Step())
            torch.cuda.synchronize()
        finally:
            ops.TC_ATTENTION = True
        assert int(fault_dev[0]) == 0
        # the first arm must have run the tcgen05 kernel (every size here is one it takes), the second not
        assert ops.calls["attn_tc"] - tc_before == (1 if tc else 0)
        outs[tc] = got.cpu().float()
        valid = row_slot >= 0
        torch.testing.assert_close(outs[tc][valid], want.float()[valid], rtol=2e-2, atol=2e-2)
    if window is None:
        # the far key wins for head 0 of the deep portion: its value row comes out
        v_far = ref.cache_row_inverse(plane[pg, 1, 0, far % page], far).float()
        torch.testing.assert_close(outs[True][:300, :hd], v_far.expand(300, hd), rtol=5e-2, atol=5e-2)
    assert bool((outs[True][400:402] == 0).all()), "padding rows inside a tile are written as zeros"
