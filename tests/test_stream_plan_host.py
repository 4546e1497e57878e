"""The K cut points of the equal-ranges schedule (b200_sgemm_stream_plan) are pure host arithmetic on (tiles, K tiles,
CTAs): checked here without a device, against a direct restatement of "cut the tile-major sequence of K tiles into
`ctas` equal ranges" (range c begins at floor(units * c / ctas)), and through the oracle for a small problem."""
import numpy as np
import pytest


def expected_cuts(sgemm, raster, M, N, K, blk, sms, min_ktiles=2):
    bm, bn, bk = blk
    grid_m, grid_n = -(-M // bm), -(-N // bn)
    tiles = grid_m * grid_n
    kts = -(-K // bk)
    ctas = min(sms, tiles * kts // min_ktiles)
    if ctas <= tiles:
        return None
    units = tiles * kts
    cuts = [[] for _ in range(tiles)]
    for c in range(1, ctas):
        u = units * c // ctas
        pos, k = divmod(u, kts)  # position in the order the kernel walks the tiles, K tile inside that tile
        if k:
            tile_m, tile_n = sgemm.map_tile(raster, pos, grid_m, grid_n)
            cuts[tile_m * grid_n + tile_n].append(k * bk)
    return cuts


SHAPES = [(1024, 1024, 1024), (1024, 1024, 16384), (512, 768, 2048), (384, 200, 4100), (130, 70, 1000), (128, 128, 64),
          (256, 256, 256), (640, 128, 8192)]


@pytest.mark.parametrize("sms", [148, 132, 7])
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_cut_points_are_the_equal_ranges(sgemm, shape, sms):
    M, N, K = shape
    # the table's kernel for the 1024-cube entries is the 128 x 128 x 32 warp-specialised one with split_k 0
    p, v = sgemm.select_config(1024, 1024, 1024, 0, 0, 0)
    assert p.pipeline >= 1 and p.split_k == 0
    blk, offs, bnd = sgemm.stream_plan(0, 0, 0, M, N, K, v, -1, sms)
    want = expected_cuts(sgemm, p.raster, M, N, K, blk, sms)
    if want is None:
        assert offs is None
        return
    assert offs is not None and len(offs) == len(want) + 1 and offs[0] == 0
    for t, w in enumerate(want):
        assert list(bnd[offs[t]:offs[t + 1]]) == w, t
    assert offs[-1] == len(bnd) == sum(len(w) for w in want)
    assert all(0 < b < K and b % blk[2] == 0 for b in bnd)


def test_pieces_restate_a_planned_problem(sgemm, orc):
    """The oracle evaluated with the reported cut points differs from the single chain only by the order of the sums
    (both stay within the float64 bound), and equals the split-K restatement when every tile has the same cut."""
    M, N, K = 128, 256, 256  # 2 tiles x 8 K tiles on 4 CTAs: every tile is cut in the middle
    p, v = sgemm.select_config(1024, 1024, 1024, 0, 0, 0)
    blk, offs, bnd = sgemm.stream_plan(0, 0, 0, M, N, K, v, -1, 4)
    assert list(offs) == [0, 1, 2] and list(bnd) == [128, 128]
    A, B = orc.fill_ab(5, 0, 0, M, N, K)
    pieces = orc.sgemm_fma_pieces(0, 0, 0, A, B, M, N, K, blk[0], blk[1], offs, bnd)
    halves = orc.sgemm_fma(0, 0, 0, A, B, M, N, K, splits=2, k_align=blk[2])
    assert np.array_equal(pieces.view(np.uint32), halves.view(np.uint32))
    ref = orc.sgemm_f64(0, 0, 0, A, B, M, N, K)
    assert orc.error_metrics(0, pieces, ref, M, N)["max_rel"] <= 1e-5 * np.sqrt(K)
