"""The layout of a step's metadata (CPU): the list-based fast path for decode-only steps
gives word for word what the general layout gives, and tiles cover every row once."""
import numpy as np
import pytest

from tiny_inference_server_b200.engine.batch import StepEntry, layout_decode, layout_step
from tiny_inference_server_b200.kernels.attention_plan import plan_tiles, planner


@pytest.mark.parametrize("n,pad", [(1, 1), (5, 8), (8, 8), (3, 4)])
def test_decode_layout_equals_general_layout(n, pad):
    entries = [StepEntry(i, [5 + i], [0]) for i in range(n)]
    starts = [0, 1, 2, 4000, 17, 33, 2, 900][:n]
    a = layout_step(entries, starts, [0, 1, 2], 49152, pad_to=pad, planners=[planner(4), planner(32)], want_all=True,
                    max_position=4095)
    b = layout_decode(entries, starts, [0, 1, 2], 49152, pad, [planner(4), planner(32)], max_position=4095)
    assert a.offsets == b.offsets and list(a.flat) == list(b.flat)
    assert a.plan_facts == b.plan_facts and a.n == b.n and a.max_position == b.max_position and b.decode_only


def test_lagging_stages_mask_negative_positions():
    lay = layout_step([StepEntry(3, [1, 2, 3, 4], [3]), StepEntry(1, [9], [0])], [0, 50], [0, 1, 2], 100, planners=[planner(2)])
    def arr(name):
        a, k = lay.offsets[name]
        return list(lay.flat[a:a + k])
    assert arr("positions") == [0, 1, 2, 3, 50] and arr("slots") == [3, 3, 3, 3, 1]
    assert arr("pos1") == [0, 0, 1, 2, 49] and arr("slot1") == [-1, 3, 3, 3, 1]
    assert arr("pos2") == [0, 0, 0, 1, 48] and arr("slot2") == [-1, -1, 3, 3, 1]
    assert arr("last") == [3, 3, 3, 3, 4] and arr("want") == [3, 4]


@pytest.mark.parametrize("g", [1, 2, 3, 4, 8, 16, 20, 64])
def test_tiles_cover_every_row_once(g):
    segs = [(0, 1), (1, 200), (201, 3), (204, 16), (220, 1), (221, 65), (286, 300)]
    keys, rows, wide, rows_in_wide = plan_tiles(segs, g)
    seen = np.zeros(586, dtype=int)
    for r0, n in keys:
        assert n * g <= 16
        seen[r0:r0 + n] += 1
    for r0, n in rows:
        assert n * g <= 64 or n == 1
        seen[r0:r0 + n] += 1
    assert (seen == 1).all()
    # the wide tiles cover the long segments once more, and exactly the leading rows tiles
    again = np.zeros(586, dtype=int)
    for r0, n in wide:
        assert 0 < n <= 128
        again[r0:r0 + n] += 1
    lead = np.zeros(586, dtype=int)
    for r0, n in rows[:rows_in_wide]:
        lead[r0:r0 + n] += 1
    assert (again == lead).all()
    for r0, n in segs:
        assert again[r0:r0 + n].sum() == (n if n >= 64 and not (g <= 16 and n * g <= 16) else 0)


def test_token_ids_outside_the_vocabulary_are_refused():
    with pytest.raises(ValueError, match="outside the vocabulary"):
        layout_step([StepEntry(0, [5, 100], [])], [0], [0], 100)
    with pytest.raises(ValueError, match="outside the vocabulary"):
        layout_decode([StepEntry(0, [-1], [0])], [0], [0], 100, 1, [planner(4)])
    with pytest.raises(ValueError, match="wanted place"):
        layout_step([StepEntry(0, [5, 6], [2])], [0], [0], 100)
