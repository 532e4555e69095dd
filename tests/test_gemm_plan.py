"""Work decomposition of the persistent int8 GEMM (h3b_gemm_i8_plan, evaluated on the host): every k-block of every tile
is covered exactly once, a tile's slices sit in the last wave on distinct pairs, slice 0 exists for every cut tile, and
the library's own choice cuts only where its estimate says it pays."""
import ctypes as C

import pytest


@pytest.fixture(scope="module")
def lib():
    import h3c_b200
    return h3c_b200.load()


def plan(lib, tiles, pairs, k_blocks, mode):
    tot, first, split = C.c_int(), C.c_int(), C.c_int()
    assert lib.h3b_gemm_i8_plan(tiles, pairs, k_blocks, mode, 1 << 40, C.byref(tot), C.byref(first), C.byref(split),
                                None, None, None, None) == 1
    items = []
    for i in range(tot.value):
        t, a, b, s = C.c_int(), C.c_int(), C.c_int(), C.c_int()
        assert lib.h3b_gemm_i8_plan(tiles, pairs, k_blocks, mode, i, None, None, None, C.byref(t), C.byref(a), C.byref(b),
                                    C.byref(s)) == 1
        items.append((t.value, a.value, b.value, s.value))
    # past the last item: refused when item outputs are asked for
    t = C.c_int()
    assert lib.h3b_gemm_i8_plan(tiles, pairs, k_blocks, mode, tot.value, None, None, None, C.byref(t), None, None, None) == 0
    return tot.value, first.value, split.value, items


@pytest.mark.parametrize("tiles,pairs,k_blocks", [(300, 74, 24), (300, 74, 96), (600, 74, 96), (1188, 74, 96), (80, 74, 4),
                                                   (900, 74, 24), (2364, 74, 24), (74, 74, 24), (75, 74, 3), (10, 74, 24),
                                                   (149, 74, 2), (300, 37, 96), (5, 2, 7)])
@pytest.mark.parametrize("mode", [0, 1, 2, 3, 5, 12, 16, 40])
def test_every_k_block_once(lib, tiles, pairs, k_blocks, mode):
    total, first, split, items = plan(lib, tiles, pairs, k_blocks, mode)
    cover = {}
    for idx, (tile, kb0, kb1, sl) in enumerate(items):
        assert 0 <= tile < tiles and 0 <= kb0 < kb1 <= k_blocks
        for kb in range(kb0, kb1):
            assert (tile, kb) not in cover
            cover[(tile, kb)] = idx
    assert len(cover) == tiles * k_blocks
    if mode == 0 or split == 1:
        assert (total, first, split) == (tiles, tiles, 1)
        return
    rem = tiles % pairs
    # only a short last wave of more than one wave is cut, into slices that fit that wave
    assert tiles > pairs and 0 < rem <= pairs // 2
    assert first == tiles - rem and first % pairs == 0 and total == first + rem * split
    assert 2 <= split <= 16 and rem * split <= pairs and split <= k_blocks // 2
    if mode >= 2:
        assert split == min(mode, pairs // rem, k_blocks // 2, 16)
    tail = items[first:]
    assert len({i % pairs for i in range(first, total)}) == len(tail)          # one tail item per pair
    for slot in range(rem):
        slices = tail[slot * split:(slot + 1) * split]
        assert [s for _, _, _, s in slices] == list(range(split))              # slice 0 (the owner) first
        assert {t for t, _, _, _ in slices} == {first + slot}
        assert all(b - a >= 2 for _, a, b, _ in slices)
        assert slices[0][1] == 0 and slices[-1][2] == k_blocks
        assert all(slices[i][2] == slices[i + 1][1] for i in range(split - 1))


def test_the_estimate_cuts_deep_tiles_only(lib):
    """On 74 pairs: the 3,072-deep projections of a 6,280-row shard (24 k-blocks) stay whole, the 12,288-deep one (96) is
    cut in four; a full last wave or a single wave is never cut."""
    assert plan(lib, 300, 74, 24, 1)[2] == 1
    assert plan(lib, 300, 74, 96, 1)[2] == 4
    assert plan(lib, 600, 74, 96, 1)[2] == 4       # 8 tail tiles: 4 x 8 = 32 slices
    assert plan(lib, 2364, 74, 96, 1)[2] == 1      # 70 tail tiles: more than half a wave
    assert plan(lib, 60, 74, 96, 1)[2] == 1        # a single wave
    assert plan(lib, 148, 74, 96, 1)[2] == 1       # full waves
