"""Work schedule of the two-SM GEMM (whole tiles round robin + stream-K tail), enumerated on the host through the
test hook ``oob_test_pair_schedule`` (the kernel runs the same code on the device).

Checked for many shapes and pair counts: every (tile, K block) is computed exactly once; a pair parks at most one
partial accumulator; the number of parts the kernel expects for a tile is the number of pairs that
really contribute; the fused modes' tile orders are permutations of the tile grid."""
import ctypes

import pytest

from ooverlap_b200 import _lib

PLAIN, AR, RS, AG = range(4)


def schedule(mode, M, N, K, pairs, stream_k, world=1, rank=0):
    lib = _lib.lib()
    cap = 9 * (4 * ((M + 255) // 256) * ((N + 255) // 256) + 8 * pairs + 64)
    buf = (ctypes.c_int * cap)()
    n = lib.oob_test_pair_schedule(mode, M, N, K, pairs, stream_k, world, rank, buf, cap)
    assert n >= 0
    return [tuple(buf[i * 9:(i + 1) * 9]) for i in range(n)]


SHAPES = [(512, 8192, 8192), (2048, 8192, 8192), (8192, 8192, 8192), (4096, 3584, 8192), (4096, 8192, 3584),
          (300, 520, 1024), (256, 256, 64), (1024, 1024, 4096), (2304, 768, 2048), (128 * 9, 256 * 5, 8192)]


@pytest.mark.parametrize("pairs", [74, 70, 66, 7, 3, 2, 1])
@pytest.mark.parametrize("stream_k", [0, 1, -1])
def test_every_k_block_of_every_tile_is_computed_once(pairs, stream_k):
    for M, N, K in SHAPES:
        items = schedule(PLAIN, M, N, K, pairs, stream_k)
        tm, tn, nkb = (M + 255) // 256, (N + 255) // 256, (K + 63) // 64
        cover = {}
        slots = set()
        per_pair = {}
        for p, seq, mb, nb, kb0, kb1, slot, parts, first in items:
            assert 0 <= mb < tm and 0 <= nb < tn and 0 <= kb0 < kb1 <= nkb
            key = (mb, nb)
            cover.setdefault(key, []).append((kb0, kb1, p, slot, parts, first))
            per_pair.setdefault(p, []).append((seq, kb0, kb1, slot))
            if slot >= 0:
                assert slot not in slots, "a workspace slot is written by one item only"
                assert slot == p and kb0 > 0
                slots.add(slot)
                assert kb1 - kb0 < nkb
            elif slot == -2:  # the part that starts a tile: its pair owns the tile and parks nothing
                assert kb0 == 0 and kb1 < nkb
            else:
                assert kb0 == 0 and kb1 == nkb
        assert len(cover) == tm * tn, (M, N, K, pairs, stream_k)
        for key, parts_list in cover.items():
            parts_list.sort()
            pos = 0
            for kb0, kb1, p, slot, parts, first in parts_list:
                assert kb0 == pos
                pos = kb1
            assert pos == nkb
            if len(parts_list) > 1:
                # what the summing warp assumes: consecutive pairs starting at `first`, head part first
                contributors = [p for _, _, p, _, _, _ in parts_list]
                assert all(x[4] == len(parts_list) for x in parts_list)
                assert all(x[5] == contributors[0] for x in parts_list)
                assert contributors == list(range(contributors[0], contributors[0] + len(parts_list)))
        # a pair's partial items: at most one that does not start a tile and one that does, whole tiles come first
        for p, lst in per_pair.items():
            assert len([x for x in lst if x[3] >= 0]) <= 1 and len([x for x in lst if x[3] == -2]) <= 1
            # the parked part comes before the owned part in the pair's order (the owner of a tile never waits for a
            # pair that is itself waiting: parked parts are computed right after the whole tiles)
            kinds = [x[3] for x in lst if x[3] != -1 or True]
            if any(k >= 0 for k in kinds) and -2 in kinds:
                assert min(i for i, k in enumerate(kinds) if k >= 0) < kinds.index(-2)
            whole_before = [i for i, k in enumerate(kinds) if k == -1]
            parked = [i for i, k in enumerate(kinds) if k >= 0]
            if parked and whole_before:
                # whole tiles dealt round robin come first; at most one whole tile lies inside the tail range
                assert len([i for i in whole_before if i > parked[0]]) <= 1


def test_stream_k_balances_the_last_wave():
    """With a tail, the K blocks per pair differ by at most one tile's worth of rounding; without it, by a whole tile."""
    for M, N, K in [(512, 8192, 8192), (2048, 8192, 8192), (4096, 3584, 8192)]:
        nkb = K // 64
        for pairs in (74, 70):
            load = {}
            for p, seq, mb, nb, kb0, kb1, slot, parts, first in schedule(PLAIN, M, N, K, pairs, 1):
                load[p] = load.get(p, 0) + kb1 - kb0
            assert len(load) == pairs and max(load.values()) - min(load.values()) <= 1, (M, N, K, pairs)
            load = {}
            for p, seq, mb, nb, kb0, kb1, slot, parts, first in schedule(PLAIN, M, N, K, pairs, -1):
                load[p] = load.get(p, 0) + kb1 - kb0
            tiles = ((M + 255) // 256) * ((N + 255) // 256)
            if tiles % pairs:
                assert max(load.values()) - min(load.get(p, 0) for p in range(pairs)) == nkb


def test_auto_rule_picks_a_tail_only_where_it_pays():
    # 8192^3 on 74 pairs wastes 1.2 % of the last wave: whole tiles only; 2048 rows waste 13 % and have a whole wave:
    # tail; 512 rows are less than a wave of tiles with operands beyond L2: whole tiles (measured slower with a tail);
    # the all-gather shape's operands fit L2: tail
    assert all(s[6] == -1 for s in schedule(PLAIN, 8192, 8192, 8192, 74, 0))
    assert any(s[6] >= 0 for s in schedule(PLAIN, 2048, 8192, 8192, 74, 0))
    assert all(s[6] == -1 for s in schedule(PLAIN, 512, 8192, 8192, 74, 0))
    assert any(s[6] >= 0 for s in schedule(PLAIN, 4096, 3584, 8192, 74, 0))
    assert any(s[6] >= 0 for s in schedule(PLAIN, 512, 2048, 2048, 74, 0))
    # shallow K (tensor-parallel shards) is never cut
    assert all(s[6] == -1 for s in schedule(PLAIN, 2048, 8192, 512, 74, 0))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_orders_are_permutations(world):
    for mode in (AR, RS, AG):
        for M, N, K in [(256 * world * 2, 768, 256), (4096, 8192, 3584), (128 * world, 512, 128)]:
            for rank in (0, world - 1):
                items = schedule(mode, M, N, K, 5, -1, world, rank)
                tm, tn = (M + 255) // 256, (N + 255) // 256
                seen = {(mb, nb) for _, _, mb, nb, *_ in items}
                assert len(items) == tm * tn and len(seen) == tm * tn
    # reduce-scatter: consecutive row blocks of the order belong to consecutive owners (when rows split evenly)
    items = sorted(schedule(RS, 4096, 8192, 3584, 64, -1, 8, 0), key=lambda x: x[1])
    owners = [mb * 256 // 512 for _, _, mb, nb, *_ in items if nb == 0]
    assert owners[:8] == list(range(8))
    # all-gather: a rank starts with its own rows
    items = sorted(schedule(AG, 4096, 3584, 8192, 64, -1, 8, 3), key=lambda x: x[1])
    assert items[0][2] * 256 // 512 == 3
