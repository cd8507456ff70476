"""The cache manager on the CPU: no page is lost, held twice or freed twice under random
orders of requests; groups with a window give pages back; state slots are zeroed."""
import random

import pytest
import torch

from tiny_inference_server_b200.cache import CacheError, CacheManager, OutOfPages, PagePool
from tiny_inference_server_b200.parts.base import KVSpec, StateSpec


def _manager(num_pages=24, page=4, slots=5, window=None, max_pos=200):
    specs = [KVSpec(2, 16), KVSpec(2, 16), KVSpec(2, 16, lag=1)]
    if window:
        specs += [KVSpec(2, 16, window=window), KVSpec(2, 16, window=window, lag=2)]
    specs.append(None)       # an entry that reads another entry's plane has no plane of its own
    return CacheManager(specs, {"pending": StateSpec((8,), torch.float32)}, page_size=page, num_pages=num_pages,
                        max_slots=slots, max_positions=max_pos, dtype=torch.float32, device="cpu")


def test_page_pool_refuses_double_free_and_foreign_ids():
    pool = PagePool(3)
    a, b = pool.allocate(), pool.allocate()
    pool.release(a)
    with pytest.raises(CacheError, match="twice"):
        pool.release(a)
    with pytest.raises(CacheError, match="outside"):
        pool.release(7)
    c, d = pool.allocate(), pool.allocate()
    assert sorted([b, c, d]) == [0, 1, 2]
    with pytest.raises(OutOfPages):
        pool.allocate()
    pool.check()


def test_groups_are_formed_by_need():
    m = _manager(window=6)
    assert len(m.groups) == 2
    assert m.groups[0].window is None and m.groups[0].num_planes == 3 and m.groups[0].max_lag == 1
    assert m.groups[1].window == 6 and m.groups[1].num_planes == 2 and m.groups[1].max_lag == 2
    assert [None if r is None else (r.group, r.index) for r in m.plane_refs] == \
        [(0, 0), (0, 1), (0, 2), (1, 0), (1, 1), None]
    assert m.groups[0].pages.shape == (3, 24, 2, 2, 4, 16)


def test_extend_allocates_whole_pages_and_release_returns_them():
    m = _manager()
    s = m.admit()
    assert m.extend(s, 1) == 0 and m.pages_held(s) == 1
    assert m.extend(s, 3) == 1 and m.pages_held(s) == 1
    assert m.extend(s, 1) == 4 and m.pages_held(s) == 2
    assert m.pages_needed(s, 3) == 0 and m.pages_needed(s, 4) == 1
    m.check()
    m.release(s)
    assert m.drained()
    with pytest.raises(CacheError, match="not live"):
        m.release(s)
    with pytest.raises(CacheError, match="not live"):
        m.extend(s, 1)


def test_out_of_pages_changes_nothing():
    m = _manager(num_pages=3, window=6)
    s = m.admit()
    m.extend(s, 8)
    before = (m.free_pages(), m.length[s], [g.held(s) for g in m.groups])
    with pytest.raises(OutOfPages):
        m.extend(s, 9)           # the full group would need 3 more pages, 1 is free
    assert (m.free_pages(), m.length[s], [g.held(s) for g in m.groups]) == before
    m.check()


def test_window_gives_pages_back_once_every_plane_has_passed_them():
    page, W = 4, 6
    m = _manager(num_pages=40, page=page, window=W)
    s = m.admit()
    full, win = m.groups
    for step in range(60):
        start = m.extend(s, 1)
        # the lagging plane (lag 2) at this step reads keys from start-2-W+1 on
        lowest = max(0, start - 2 - W + 1)
        assert win.first[s] == lowest // page
        assert win.end[s] == start // page + 1
        assert full.first[s] == 0
        for lp in range(win.first[s], win.end[s]):
            assert win.table_host[s, lp] >= 0
        for lp in range(0, win.first[s]):
            assert win.table_host[s, lp] == -1
    assert win.held(s) <= (W + 2) // page + 2
    assert full.held(s) == 15
    m.check()
    m.release(s)
    assert m.drained()


def test_state_slots_are_zeroed_on_admission():
    m = _manager()
    s = m.admit()
    m.states["pending"][s] = 7.0
    m.release(s)
    s2 = m.admit()
    assert s2 == s and float(m.states["pending"][s2].abs().sum()) == 0.0


def test_slots_run_out():
    m = _manager(slots=2)
    m.admit(), m.admit()
    assert not m.has_free_slot()
    with pytest.raises(CacheError, match="no free request slot"):
        m.admit()


@pytest.mark.parametrize("seed", range(6))
@pytest.mark.parametrize("window", [None, 6])
def test_random_orders_keep_the_invariants(seed, window):
    rng = random.Random(seed)
    m = _manager(num_pages=30, page=4, slots=5, window=window, max_pos=120)
    for g in m.groups:
        g.pool.shuffle(rng)
    live = []
    for _ in range(600):
        op = rng.random()
        if op < 0.2 and m.has_free_slot():
            live.append(m.admit())
        elif op < 0.8 and live:
            s = rng.choice(live)
            n = rng.choice([1, 1, 1, 2, 5, 9, 17])
            if m.length[s] + n > m.max_positions:
                continue
            need = m.pages_needed(s, n)
            try:
                m.extend(s, n)
                assert need <= 30
            except OutOfPages:
                assert need > m.free_pages() or window is not None
        elif op < 0.9 and live:
            s = rng.choice(live)
            try:
                m.truncate(s, rng.randint(max(0, m.length[s] - 3), m.length[s]))
            except CacheError:
                assert window is not None
        elif live:
            s = live.pop(rng.randrange(len(live)))
            m.release(s)
        m.check()
    for s in live:
        m.release(s)
    m.check()
    assert m.drained()
    for g in m.groups:
        assert (g.table_host == -1).all()
