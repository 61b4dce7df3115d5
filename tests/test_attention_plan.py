"""The attention work lists of a step (CPU): every token is planned once, a decoded token's
splits are the ones its own position and window give, whatever else is in the batch."""
import random

import numpy as np
import pytest

from lockstep_b200.engine.batch import plan_attention


def random_portions(rng, n):
    portions, off = [], 0
    for slot in range(n):
        length = rng.choice([1, 1, 1, 2, 5, 16, 17, 130, 300])
        start = rng.randrange(0, 2000)
        portions.append((slot, off, start, length))
        off += length
    return portions, off


@pytest.mark.parametrize("window", [0, 100, 700])
@pytest.mark.parametrize("split_size,tile_tokens", [(256, 16), (256, 128), (64, 16)])
def test_every_token_is_planned_once(window, split_size, tile_tokens):
    rng = random.Random(window * 7 + split_size + tile_tokens)
    for _ in range(30):
        portions, total = random_portions(rng, rng.randrange(1, 6))
        tile, split, combine, n_slots = plan_attention(portions, window, split_size, tile_tokens)
        seen = np.zeros(total, dtype=np.int32)
        by_offset = {}
        for slot, off, start, length in portions:
            for i in range(length):
                by_offset[off + i] = (slot, start + i, length)
        for slot, off, ntok, pos0, s_lo, s_hi, scratch, _ in tile.tolist():
            assert 1 <= ntok <= tile_tokens and scratch == -1
            for i in range(ntok):
                want_slot, pos, length = by_offset[off + i]
                assert (want_slot, pos) == (slot, pos0 + i) and length > 1
                seen[off + i] += 1
            # the splits a tile walks reach from its first row's first key to its last row's last key
            lo = max(0, pos0 - window + 1) if window else 0
            assert s_lo == lo // split_size and s_hi == (pos0 + ntok - 1) // split_size + 1
        used = np.zeros(n_slots, dtype=np.int32)
        for off, first, ntok, count in combine.tolist():
            slot, pos, length = by_offset[off]
            assert length == 1 and ntok == 1
            seen[off] += 1
            lo = max(0, pos - window + 1) if window else 0
            want = list(range(lo // split_size, pos // split_size + 1))
            rows = [r for r in split.tolist() if r[6] in range(first, first + count)]
            # its splits, ascending, in scratch slots side by side: the fold's order
            assert [r[4] for r in rows] == want and [r[6] for r in rows] == list(range(first, first + count))
            assert all(r[0] == slot and r[1] == off and r[3] == pos and r[5] == r[4] + 1 for r in rows)
            used[first:first + count] += 1
        assert (seen == 1).all() and (used == 1).all() and len(split) == n_slots


def test_the_longest_contexts_come_first():
    portions = [(0, 0, 0, 300), (1, 300, 900, 40), (2, 340, 5, 1)]
    tile, _, _, _ = plan_attention(portions, 0, 256, 128)
    ends = [int(r[3] + r[2]) for r in tile]
    assert ends == sorted(ends, reverse=True) and len(tile) == 4


def test_a_token_is_planned_alike_in_any_batch():
    alone = plan_attention([(3, 0, 777, 1)], 100, 256)
    among = plan_attention([(0, 0, 10, 20), (3, 20, 777, 1), (1, 21, 5000, 1)], 100, 256)
    mine = [r for r in among[1].tolist() if r[0] == 3]
    # the same splits of the same position; only the token's offset and its scratch slots move
    assert [(r[3], r[4], r[5]) for r in mine] == [(r[3], r[4], r[5]) for r in alone[1].tolist()]
