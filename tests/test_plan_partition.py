"""Index arithmetic of the compiled product plan, checked on the CPU.

The persistent kernel splits a group's tiles (row tile x k tile) over the CTAs as contiguous
ranges -- whole row tiles when there is at least one per CTA, else an even deal of tiles -- and
hands row tiles that straddle CTAs through numbered parts. This file restates that
arithmetic (plan_lo / plan_owner / plan_parts of nn_b200/csrc/plan.cuh) and checks, for the
benchmark shapes and for awkward ones, that every tile is owned exactly once, that every split row
tile gets exactly the parts 0..n-1, and that the library's nnq_plan_geometry bounds hold."""
import pytest

from nn_b200 import plan

WARPS = 16


def lo(c, nc, row_tiles, kt):
    if row_tiles >= nc:          # whole row tiles per CTA
        return ((c * row_tiles) // nc) * kt
    return (c * row_tiles * kt) // nc


def owner(i, nc, tiles):
    return ((i + 1) * nc - 1) // tiles


def parts_of(rt, kt, tiles, nc, c, lo_c):
    if tiles >= nc:
        first, last = owner(rt * kt, nc, tiles), owner((rt + 1) * kt - 1, nc, tiles)
        return last - first + 1, c - first
    return kt, lo_c - rt * kt


SHAPES = [
    # (row tiles, k tiles): Qwen3-8B groups (q/k/v, o, gate/up, down) and their 1/2, 1/4, 1/8 shards
    (384, 16), (256, 16), (1536, 16), (256, 48),
    (192, 16), (256, 8), (768, 16), (256, 24),
    (48, 16), (256, 2), (192, 16), (256, 6),
    # Qwen3-32B shapes, the vocabulary projection, and degenerate cases
    (640, 20), (320, 32), (3200, 20), (320, 100), (9496, 16),
    (1, 1), (1, 100), (3, 7), (5, 29), (147, 1), (148, 1), (149, 1), (2, 74), (1, 147), (1, 149),
]


@pytest.mark.parametrize("row_tiles,kt", SHAPES)
@pytest.mark.parametrize("nc", [148, 132, 7, 1])
def test_partition_covers_every_tile_once_and_parts_are_complete(row_tiles, kt, nc):
    tiles = row_tiles * kt
    max_tiles, pmax = plan.geometry(row_tiles, kt, nc)
    seen = [0] * tiles
    contributions = {}   # row tile -> list of (part, parts) handed in by CTAs that do not hold it whole
    direct = set()
    for c in range(nc):
        a, b = lo(c, nc, row_tiles, kt), lo(c + 1, nc, row_tiles, kt)
        assert 0 <= a <= b <= tiles
        assert b - a <= max_tiles
        # warps take tiles a + w, a + w + 16, ...: together exactly [a, b), slot = i - a
        mine = sorted(i for w in range(WARPS) for i in range(a + w, b, WARPS))
        assert mine == list(range(a, b))
        for i in mine:
            seen[i] += 1
            if row_tiles < nc:
                assert owner(i, nc, tiles) == c
            assert 0 <= i - a < max_tiles
        if a == b:
            continue
        for rt in range(a // kt, (b - 1) // kt + 1):
            s, e = max(a, rt * kt), min(b, (rt + 1) * kt)
            assert s < e
            if s == rt * kt and e == (rt + 1) * kt:
                direct.add(rt)
            else:
                assert row_tiles < nc, "with a row tile per CTA nothing straddles CTAs"
                n, p = parts_of(rt, kt, tiles, nc, c, a)
                assert 0 <= p < n <= pmax
                contributions.setdefault(rt, []).append((p, n))
    assert all(v == 1 for v in seen)
    for rt in range(row_tiles):
        if rt in direct:
            assert rt not in contributions
            continue
        got = contributions[rt]
        n = got[0][1]
        assert all(x[1] == n for x in got)
        assert sorted(x[0] for x in got) == list(range(n)), (rt, got)


def test_geometry_rejects_bad_arguments():
    from nn_b200 import api
    with pytest.raises(api.InvalidArgument):
        plan.geometry(0, 16, 148)
    with pytest.raises(api.InvalidArgument):
        plan.geometry(1 << 20, 1 << 10, 148)
