"""The attention kernels against the upstream project's own Triton kernels, run unchanged on the
GPU on the same queries, keys and values.

``paged_flash_decode`` (upstream paged_attention_kernels.py:207-261) and
``triton_intradoc_attention`` (upstream intradocatt_fwd_kernels.py:158-169) are imported from a
copy of the upstream checkout (``baseline/_ref`` at the repository root, or the folder named by
``TIS_UPSTREAM``); nothing of them is rebound.  This pins on upstream's own output what
``tests/golden`` pins only through a stand-in: the score scale, the causal rule and which kv head a
query head reads.  Cases and tolerance are upstream's: decode rows over scattered pages at context
lengths 37 / 512 / 2000 with ``allclose(rtol=1e-2, atol=1e-2)`` and a wrong-group negative
control (test_gqa_paged.py:15-53); packed prompts of 7 / 33 / 18 / 1 / 2 tokens
(test_server.py:66-87).  The two pools have different layouts (upstream
``[layer, kv head, 2, page, token, hd]`` with plain rows; here ``[page, 2, kv head, token, hd]``
with permuted rows), so both are filled from the same logical keys and values."""
import os
import random
import sys
from collections import deque

import pytest
import torch

import kernel_refs as ref

pytestmark = pytest.mark.gpu

ROOT = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), os.pardir))


def _upstream():
    for folder in (os.environ.get("TIS_UPSTREAM"), os.path.join(ROOT, "baseline", "_ref")):
        if folder and os.path.isfile(os.path.join(folder, "paged_attention_kernels.py")):
            if folder not in sys.path:
                sys.path.insert(0, folder)
            import block_table as BT
            import intradocatt_fwd_kernels as IK
            import paged_attention_kernels as PK
            return BT, PK, IK
    pytest.skip("no copy of the upstream checkout (baseline/_ref or TIS_UPSTREAM)")


def _ops():
    from tiny_inference_server_b200.kernels import ops
    ops.library()
    return ops


@pytest.mark.parametrize("H,KVH,hd", [(8, 2, 64), (12, 3, 128)])
def test_decode_attention_equals_upstream_paged_flash_decode(H, KVH, hd):
    BT, PK, _ = _upstream()
    ops = _ops()
    dev, tpb, layer = "cuda", 16, 0
    group = H // KVH
    torch.manual_seed(0)
    pool = BT.block_table(1, KVH, hd, 64 * 1024 * 1024, tpb, dev)
    order = list(pool.free_block_queue)
    random.Random(0).shuffle(order)
    pool.free_block_queue = deque(order)
    kv_lens = [37, 512, 2000]
    max_pages = max((L + tpb - 1) // tpb for L in kv_lens)
    plane = torch.zeros(pool.num_blocks, 2, KVH, tpb, hd, dtype=torch.bfloat16)
    table = torch.full((len(kv_lens), max_pages), -1, dtype=torch.int32)
    page_ids, page_starts = [], [0]
    for s, L in enumerate(kv_lens):
        k = torch.randn(KVH, L, hd).to(torch.bfloat16)
        v = torch.randn(KVH, L, hd).to(torch.bfloat16)
        ids = [pool.allocate_block() for _ in range((L + tpb - 1) // tpb)]
        page_ids += ids
        page_starts.append(page_starts[-1] + len(ids))
        for p, pg in enumerate(ids):
            a, b = p * tpb, min(p * tpb + tpb, L)
            pool.block[layer, :, 0, pg, :b - a, :] = k[:, a:b].to(dev)       # upstream's layout (test_gqa_paged.py:26-27)
            pool.block[layer, :, 1, pg, :b - a, :] = v[:, a:b].to(dev)
            table[s, p] = pg
            for t in range(a, b):
                plane[pg, 0, :, t - a] = ref.cache_row(k[:, t], t)          # this engine's layout and row format
                plane[pg, 1, :, t - a] = ref.cache_row(v[:, t], t)
    q = torch.randn(len(kv_lens), H, hd).to(torch.bfloat16).to(dev)
    pt = torch.tensor(page_ids, dtype=torch.int32, device=dev)
    cs = torch.tensor(page_starts, dtype=torch.int32, device=dev)
    kl = torch.tensor(kv_lens, dtype=torch.int32, device=dev)
    theirs = PK.paged_flash_decode(q, pt, pool, kl, group, cs, max(kv_lens), layer)

    fault = torch.zeros(4, dtype=torch.int32, device=dev)
    positions = torch.tensor([L - 1 for L in kv_lens], dtype=torch.int32, device=dev)
    slots = torch.arange(len(kv_lens), dtype=torch.int32, device=dev)
    ours = ops.paged_attention(q.reshape(len(kv_lens), H * hd).contiguous(),
                               torch.empty(len(kv_lens), H * hd, dtype=torch.bfloat16, device=dev), plane.to(dev),
                               table.to(dev), positions, slots, H, KVH, hd, tpb, None, fault).view(len(kv_lens), H, hd)
    assert int(fault[0]) == 0
    assert torch.allclose(theirs.float(), ours.float(), rtol=1e-2, atol=1e-2), \
        f"max difference {float((theirs.float() - ours.float()).abs().max())}"
    # upstream's negative control (a wrong group size reads other kv heads and must not match).  Upstream
    # passes the number of kv heads, which makes its kernel index kv heads past the pool; twice the group
    # size is wrong as well and stays inside it.
    wrong = PK.paged_flash_decode(q, pt, pool, kl, 2 * group, cs, max(kv_lens), layer)
    assert not torch.allclose(wrong.float(), ours.float(), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("H,KVH,hd", [(4, 2, 64), (12, 3, 128)])
@pytest.mark.parametrize("lens", [[7, 33, 18, 1, 2], [200, 70, 3]])
def test_prompt_attention_equals_upstream_intradoc_attention(H, KVH, hd, lens):
    _, _, IK = _upstream()
    ops = _ops()
    dev, page = "cuda", 16
    group = H // KVH
    g = torch.Generator().manual_seed(1)
    T = sum(lens)
    q = torch.randn(T, H, hd, generator=g).to(torch.bfloat16)
    k = torch.randn(T, KVH, hd, generator=g).to(torch.bfloat16)
    v = torch.randn(T, KVH, hd, generator=g).to(torch.bfloat16)
    cuseq = [0]
    for L in lens:
        cuseq.append(cuseq[-1] + L)
    theirs, _ = IK.triton_intradoc_attention(q.to(dev), k.to(dev), v.to(dev),
                                             torch.tensor(cuseq, dtype=torch.int32, device=dev), max(lens), group)

    max_pages = max((L + page - 1) // page for L in lens)
    num_pages = len(lens) * max_pages
    perm = torch.randperm(num_pages, generator=g).tolist()
    plane = torch.zeros(num_pages, 2, KVH, page, hd, dtype=torch.bfloat16)
    table = torch.full((len(lens), max_pages), -1, dtype=torch.int32)
    slots, positions = [], []
    for s, L in enumerate(lens):
        for t in range(L):
            if t % page == 0:
                table[s, t // page] = perm.pop()
            pg = int(table[s, t // page])
            plane[pg, 0, :, t % page] = ref.cache_row(k[cuseq[s] + t], t)
            plane[pg, 1, :, t % page] = ref.cache_row(v[cuseq[s] + t], t)
            slots.append(s)
            positions.append(t)
    fault = torch.zeros(4, dtype=torch.int32, device=dev)
    ours = ops.paged_attention(q.reshape(T, H * hd).to(dev), torch.empty(T, H * hd, dtype=torch.bfloat16, device=dev),
                               plane.to(dev), table.to(dev), torch.tensor(positions, dtype=torch.int32, device=dev),
                               torch.tensor(slots, dtype=torch.int32, device=dev), H, KVH, hd, page, None,
                               fault).view(T, H, hd)
    assert int(fault[0]) == 0
    assert torch.allclose(theirs.float(), ours.float(), rtol=1e-2, atol=1e-2), \
        f"max difference {float((theirs.float() - ours.float()).abs().max())}"
    # negative control: upstream told twice the group size reads other kv heads (still inside k and v)
    wrong, _ = IK.triton_intradoc_attention(q.to(dev), k.to(dev), v.to(dev),
                                            torch.tensor(cuseq, dtype=torch.int32, device=dev), max(lens), 2 * group)
    assert not torch.allclose(wrong.float(), ours.float(), rtol=1e-2, atol=1e-2)
