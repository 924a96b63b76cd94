"""The host-built static deal of work items (forward and dQ pass): every item exactly once, lists balanced,
heavy lists on the first blocks so that the two blocks that share an SM carry the same total everywhere."""
import ctypes

import numpy as np
import pytest

from modern_llm_v1_b200 import _lib


def _deal(n_groups, n_qtiles, T, n_ctas, cost=1):
    ids = np.full(n_ctas * 8, 0xDEAD, dtype=np.uint16)
    per = ctypes.c_int(-7)
    rc = _lib.load().b200attn_item_deal(n_groups, n_qtiles, T, n_ctas, cost, ids.ctypes.data, ctypes.byref(per))
    assert rc == 0
    return ids, per.value


def _tiles(item, n_groups, n_qtiles, T):
    qt = n_qtiles - 1 - item // n_groups
    return (min(T, qt * 128 + 128) + 63) // 64


@pytest.mark.parametrize("B,Hq,T,n_ctas", [(32, 6, 512, 296), (8, 6, 512, 192), (3, 5, 1000, 120), (1, 7, 4000, 217),
                                           (2, 148, 128, 296)])
def test_every_item_exactly_once_and_lists_balanced(B, Hq, T, n_ctas):
    n_groups, n_qtiles = B * Hq, (T + 127) // 128
    n_items = n_groups * n_qtiles
    ids, per = _deal(n_groups, n_qtiles, T, n_ctas)
    if per == 0:
        pytest.skip("this shape does not use the table")
    lists = ids[:n_ctas * per].reshape(n_ctas, per)
    seen = lists[lists != 0xFFFF]
    assert sorted(seen.tolist()) == list(range(n_items))
    loads = []
    for row in lists:
        live = row[row != 0xFFFF]
        assert len(live) >= 1 and (row[len(live):] == 0xFFFF).all()  # items first, then the end marks
        w = [_tiles(int(i), n_groups, n_qtiles, T) for i in live]
        assert w == sorted(w, reverse=True)  # heaviest item first within a block
        loads.append(sum(w) * 2 + len(w))
    assert loads == sorted(loads, reverse=True)  # heavy lists on the low block indices
    heaviest_item = 2 * _tiles(0, n_groups, n_qtiles, T) + 1
    assert max(loads) - min(loads) <= heaviest_item  # the guarantee of longest-processing-time-first


def test_blocks_that_share_an_sm_carry_the_same_total_at_the_training_shape():
    # B=32, Hq=6, T=512 on 148 SMs x 2 blocks: block i and block i + 148 share an SM
    n_groups, n_qtiles, T = 192, 4, 512
    ids, per = _deal(n_groups, n_qtiles, T, 296)
    lists = ids[:296 * per].reshape(296, per)
    tiles = [sum(_tiles(int(i), n_groups, n_qtiles, T) for i in row[row != 0xFFFF]) for row in lists]
    assert set(tiles) == {12, 14}
    per_sm = [tiles[i] + tiles[i + 148] for i in range(148)]
    assert max(per_sm) == 26 and per_sm.count(26) >= 144


def test_shapes_outside_the_table():
    assert _deal(192, 4, 512, 297)[1] == 0      # more blocks than the table holds
    assert _deal(100, 1, 128, 296)[1] == 0      # fewer items than blocks
    assert _deal(1, 4000, 512000, 8)[1] == 0    # lists longer than eight items
    lib = _lib.load()
    assert lib.b200attn_item_deal(0, 4, 512, 296, 1, None, None) == 1
