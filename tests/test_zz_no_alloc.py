"""The decode attention entry point that allocates nothing (csrc/attention_noalloc.h).

It is meant for programs that give this library raw device pointers and cannot let it
allocate: hosts that own all device memory under a fixed budget, or loops in which a
device allocation is not allowed because it can stall the whole GPU or fail when memory
is tight.  The test calls it the way such a program would — through its exported C
symbol, with plain pointers — twice in a row, and compares with the regular entry point
(which is given scratch memory by the caller) on the same inputs.

Collected last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(seed, H, KVH, hd, page, lens, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    slots = len(lens)
    max_pages = max((L + page - 1) // page for L in lens) + 1
    num_pages = slots * max_pages + 2
    perm = torch.randperm(num_pages, generator=g)
    table = perm[: slots * max_pages].reshape(slots, max_pages).to(torch.int32)
    plane = (torch.randn(num_pages, 2, KVH, page, hd, generator=g) * 0.7).to(dtype)
    n = slots
    q = torch.randn(n, (H + 2 * KVH) * hd, generator=g).to(dtype)
    positions = torch.tensor([L - 1 for L in lens], dtype=torch.int32)
    row_slot = torch.arange(slots, dtype=torch.int32)
    return q, plane, table, positions, row_slot


def _call(lib, name, q, out, plane, table, positions, row_slot, tiles0, tilesn, H, KVH, page, per, splits, scratch, fault):
    def p(t):
        return ctypes.c_void_p(0 if t is None else t.data_ptr())
    hd = plane.shape[-1]
    n = q.shape[0]
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    scale = ctypes.c_float(1.0 / math.sqrt(hd))
    head = [p(q), q.stride(0), p(out), out.stride(0), p(plane), p(table), table.stride(0), plane.shape[0],
            p(positions), p(row_slot), p(tiles0), p(tilesn), n]
    tail = [n, H, KVH, page, 0, scale, per, splits]
    if name == "tis_attn_mma":
        return lib.tis_attn_mma(1, *head, 1, *tail, p(scratch), p(fault), stream)
    return lib.tis_attn_decode_noalloc(*head, *tail, p(fault), stream)


@pytest.mark.parametrize("H,KVH,hd,page,lens,splits", [(12, 3, 128, 16, [4000, 517, 64, 1, 2300, 999, 3, 70], 16),
                                                       (4, 2, 32, 8, [300, 45, 129], 5)])
def test_no_alloc_entry_point_matches_the_regular_one_twice(H, KVH, hd, page, lens, splits):
    from tiny_inference_server_b200.kernels import ops
    lib = ops.attention_library(hd)
    lib.tis_attn_decode_noalloc.restype = ctypes.c_int
    dev = "cuda"
    for call in range(2):                              # two calls in a row share the built-in scratch
        q, plane, table, positions, row_slot = (t.to(dev) for t in _inputs(20 + call, H, KVH, hd, page, lens))
        n = q.shape[0]
        tiles0 = torch.arange(n, dtype=torch.int32, device=dev)
        tilesn = torch.ones(n, dtype=torch.int32, device=dev)
        per = ((max(lens) + splits - 1) // splits + 63) // 64 * 64
        nsplit = (max(lens) + per - 1) // per
        fault = torch.zeros(4, dtype=torch.int32, device=dev)
        want = torch.full((n, H * hd), 3.0, dtype=torch.bfloat16, device=dev)
        scratch = torch.empty(lib.tis_attn_scratch_floats(n, H, nsplit), dtype=torch.float32, device=dev)
        assert _call(lib, "tis_attn_mma", q, want, plane, table, positions, row_slot, tiles0, tilesn, H, KVH, page,
                     per, nsplit, scratch, fault) == 0
        got = torch.full((n, H * hd), -3.0, dtype=torch.bfloat16, device=dev)
        before = torch.cuda.memory_stats()["allocation.all.allocated"]      # allocations made so far
        status = _call(lib, "tis_attn_decode_noalloc", q, got, plane, table, positions, row_slot, tiles0, tilesn, H,
                       KVH, page, per, nsplit, None, fault)
        assert status == 0, lib.tis_last_error().decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_stats()["allocation.all.allocated"] == before
        assert int(fault[0]) == 0
        torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=2e-2)
        # and both agree with the plain reference of the operation
        import kernel_refs as ref
        plain = ref.paged_attention(q.cpu(), torch.empty(n, H * hd, dtype=torch.bfloat16), plane.cpu(), table.cpu(),
                                    positions.cpu(), row_slot.cpu(), H, KVH, hd, page, None,
                                    torch.zeros(4, dtype=torch.int32))
        torch.testing.assert_close(got.cpu().float(), plain.float(), rtol=2e-2, atol=2e-2)


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    from tiny_inference_server_b200.kernels import ops
    lib = ops.attention_library(128)
    lib.tis_attn_decode_noalloc.restype = ctypes.c_int
    z = ctypes.c_void_p(0)
    # 4096 rows x 64 heads x 64 splits x 129 floats is far beyond the built-in 2 Mi floats
    status = lib.tis_attn_decode_noalloc(z, 0, z, 0, z, z, 0, 0, z, z, z, z, 4096, 4096, 64, 8, 16, 0,
                                         ctypes.c_float(1.0), 64, 64, z, z)
    assert status != 0
    msg = lib.tis_last_error().decode()
    assert "scratch" in msg and "2097152" in msg
