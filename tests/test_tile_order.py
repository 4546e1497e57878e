"""Tile orders of the kernels (row-major, banded, Hilbert) evaluated on the host through the C ABI: each
is a permutation of the tile grid, and the Hilbert order keeps consecutive tiles adjacent."""
import pytest

GRIDS = [(1, 1), (1, 7), (7, 1), (4, 4), (5, 3), (32, 32), (13, 29), (29, 13), (128, 2), (3, 100), (48, 16), (33, 33)]


@pytest.mark.parametrize("raster", [0, 1, 2])
@pytest.mark.parametrize("grid", GRIDS, ids=lambda g: f"{g[0]}x{g[1]}")
def test_order_is_a_permutation(sgemm, raster, grid):
    gm, gn = grid
    seen = set()
    for i in range(gm * gn):
        tm, tn = sgemm.map_tile(raster, i, gm, gn)
        assert 0 <= tm < gm and 0 <= tn < gn
        seen.add((tm, tn))
    assert len(seen) == gm * gn


def test_hilbert_locality(sgemm):
    # inside a power-of-two square consecutive tiles are edge neighbours
    for s in (2, 4, 8, 16, 32):
        prev = sgemm.map_tile(2, 0, s, s)
        for i in range(1, s * s):
            cur = sgemm.map_tile(2, i, s, s)
            assert abs(cur[0] - prev[0]) + abs(cur[1] - prev[1]) == 1
            prev = cur
    # a window of 148 consecutive tiles of a 32 x 32 grid (what 148 persistent CTAs work on together)
    # touches fewer distinct tile rows + columns than the banded or row-major orders
    def footprint(raster):
        worst = 0
        for start in range(0, 32 * 32 - 148, 37):
            cells = [sgemm.map_tile(raster, i, 32, 32) for i in range(start, start + 148)]
            worst = max(worst, len({c[0] for c in cells}) + len({c[1] for c in cells}))
        return worst
    assert footprint(2) <= footprint(1) <= footprint(0)


def test_bad_arguments(sgemm):
    import rocm_sgemm_b200 as pkg
    with pytest.raises(pkg.SgemmError):
        sgemm.map_tile(2, 16, 4, 4)
    with pytest.raises(pkg.SgemmError):
        sgemm.map_tile(7, 0, 4, 4)
