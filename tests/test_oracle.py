"""The CPU oracle against the committed fixtures made from the reference's own host code
(tests/golden/make_golden.py) and, where oracle/_ref is built, against that code directly."""
import json
import os

import numpy as np
import pytest

from common import LAYOUTS, bits, sha, as2d

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_init_matrix_first_value(orc):
    # mt19937(1) + U(-1,1): first draw, as the reference's init_matrix produces it
    assert orc.init_matrix(0, 2, 2)[0] == np.float32(-0.16595602)


def test_small_gemm_matches_reference_fixture(orc):
    g = np.load(os.path.join(GOLDEN, "ref_gemm_small.npz"))
    M, N, K = (int(x) for x in g["shape"])
    for la in (0, 1):
        assert np.array_equal(bits(orc.init_matrix(la, M, K)), bits(g[f"A_{la}"]))
    for lb in (0, 1):
        assert np.array_equal(bits(orc.init_matrix(lb, K, N)), bits(g[f"B_{lb}"]))
    for (la, lb, lc) in LAYOUTS:
        C = orc.sgemm_f32(lc, la, lb, g[f"A_{la}"], g[f"B_{lb}"], M, N, K)
        assert np.array_equal(bits(C), bits(g[f"C_{la}{lb}{lc}"])), (la, lb, lc)


def test_digests_at_reference_test_shapes(orc):
    with open(os.path.join(GOLDEN, "ref_gemm_digests.json")) as f:
        dig = json.load(f)
    for key, want in dig["init_matrix"].items():
        shape, lay = key.split("_")
        rows, cols = (int(x) for x in shape.split("x"))
        assert sha(orc.init_matrix(int(lay), rows, cols)) == want, key
    for key, want in dig["sgemm_cpu"].items():
        shape, lay = key.split("_")
        m, n, k = (int(x) for x in shape.split("x"))
        la, lb, lc = (int(x) for x in lay)
        A, B = orc.init_matrix(la, m, k), orc.init_matrix(lb, k, n)
        assert sha(orc.sgemm_f32(lc, la, lb, A, B, m, n, k, threads=orc.max_threads())) == want, key


def test_against_reference_build_when_present(orc):
    if not orc.have_ref():
        pytest.skip("oracle/_ref not built (reference tree absent)")
    M, N, K = 70, 45, 33  # ragged on purpose
    for (la, lb, lc) in LAYOUTS:
        A, B = orc.ref_init_matrix(la, M, K), orc.ref_init_matrix(lb, K, N)
        assert np.array_equal(bits(A), bits(orc.init_matrix(la, M, K)))
        want = orc.ref_sgemm_cpu(lc, la, lb, A, B, M, N, K)
        assert np.array_equal(bits(orc.sgemm_f32(lc, la, lb, A, B, M, N, K)), bits(want))


def test_variants_agree_with_numpy(orc):
    M, N, K = 37, 29, 301
    A, B = orc.fill_ab(7, 0, 1, M, N, K)
    A2, B2 = as2d(A, 0, M, K).astype(np.float64), as2d(B, 1, K, N).astype(np.float64)
    ref = orc.sgemm_f64(1, 0, 1, A, B, M, N, K)
    assert np.allclose(as2d(ref, 1, M, N), A2 @ B2, rtol=1e-12, atol=1e-12)
    for C in (orc.sgemm_f32(1, 0, 1, A, B, M, N, K), orc.sgemm_fma(1, 0, 1, A, B, M, N, K),
              orc.sgemm_fma(1, 0, 1, A, B, M, N, K, splits=4, k_align=16)):
        e = orc.error_metrics(1, C, ref, M, N)
        assert e["max_rel"] <= 1e-5 * np.sqrt(K)
    # rows band: only the requested rows are written
    band = orc.sgemm_f32(1, 0, 1, A, B, M, N, K, rows=(5, 9))
    full = orc.sgemm_f32(1, 0, 1, A, B, M, N, K)
    assert np.array_equal(as2d(band, 1, M, N)[5:9], as2d(full, 1, M, N)[5:9])
    assert not as2d(band, 1, M, N)[:5].any() and not as2d(band, 1, M, N)[9:].any()


def test_fma_split_definition(orc):
    # the split-K restatement: slices of ceil(K/splits) rounded up to k_align, summed in order
    M, N, K = 3, 5, 100
    A, B = orc.fill_ab(11, 0, 0, M, N, K)
    C = orc.sgemm_fma(0, 0, 0, A, B, M, N, K, splits=3, k_align=16)  # slices of 48: [0,48) [48,96) [96,100)
    A2, B2 = as2d(A, 0, M, K), as2d(B, 0, K, N)
    want = np.zeros((M, N), dtype=np.float32)
    for i in range(M):
        for j in range(N):
            tot = None
            for k0 in (0, 48, 96):
                acc = np.float32(0)
                for k in range(k0, min(K, k0 + 48)):
                    # fused multiply-add in exact arithmetic, rounded once
                    acc = np.float32(np.float64(A2[i, k]) * np.float64(B2[k, j]) + np.float64(acc))
                tot = acc if tot is None else np.float32(tot + acc)
            want[i, j] = tot
    # float64 product+sum of floats is exact enough to equal the single rounding of fmaf except in
    # double-rounding corner cases; allow 1 ulp
    assert np.max(np.abs(bits(C.reshape(M, N)).astype(np.int64) - bits(want).astype(np.int64))) <= 1


def test_identity_and_pattern_fills(orc):
    I = orc.fill_identity(1, 6, 6)
    assert np.array_equal(as2d(I, 1, 6, 6), np.eye(6, dtype=np.float32))
    P = orc.fill_pattern(0, 2, 4)
    assert np.array_equal(P, np.float32([1.025, 1.05, 1.075, 1.1, 1.0, 1.025, 1.05, 1.075]))
    A, _ = orc.fill_ab(1, 0, 0, 5, 5, 5, with_b=False)
    C = orc.sgemm_fma(0, 0, 0, A, orc.fill_identity(0, 5, 5), 5, 5, 5)
    assert np.array_equal(bits(C), bits(A))


def test_fma_pieces_restates_ordered_sum_of_chains(orc):
    """Per-tile K cut points: with the same cut points in every tile the result is the split-K restatement, with no
    cut points the single chain; a tile with its own cut points differs from its neighbours only inside that tile."""
    M, N, K, bm, bn = 96, 80, 100, 32, 32
    A, B = orc.fill_ab(7, 0, 1, M, N, K)
    tiles = 3 * 3
    none = orc.sgemm_fma_pieces(0, 0, 1, A, B, M, N, K, bm, bn, np.zeros(tiles + 1, np.int32), np.zeros(0, np.int32))
    assert np.array_equal(none.view(np.uint32), orc.sgemm_fma(0, 0, 1, A, B, M, N, K).view(np.uint32))
    # one cut at 64 in every tile = sgemm_fma(splits=2, k_align=16): [0,64) [64,100); two pieces commute
    offs = np.arange(tiles + 1, dtype=np.int32)
    bnd = np.full(tiles, 64, np.int32)
    same = orc.sgemm_fma_pieces(0, 0, 1, A, B, M, N, K, bm, bn, offs, bnd)
    assert np.array_equal(same.view(np.uint32), orc.sgemm_fma(0, 0, 1, A, B, M, N, K, splits=2, k_align=16).view(np.uint32))
    # three pieces [0,48) [48,96) [96,100): the last piece's chain first, then the others in ascending K order
    offs = np.arange(tiles + 1, dtype=np.int32) * 2
    bnd = np.tile(np.array([48, 96], np.int32), tiles)
    three = orc.sgemm_fma_pieces(0, 0, 1, A, B, M, N, K, bm, bn, offs, bnd).reshape(M, N)
    a2, b2 = A.reshape(M, K), B.reshape(N, K)  # A row-major, B col-major

    def chain(i, j, k0, k1):
        acc = np.float32(0)
        for k in range(k0, k1):
            acc = np.float32(np.float64(a2[i, k]) * np.float64(b2[j, k]) + np.float64(acc))
        return acc
    for i, j in [(0, 0), (31, 33), (95, 79), (40, 7)]:
        want = np.float32(np.float32(chain(i, j, 96, K) + chain(i, j, 0, 48)) + chain(i, j, 48, 96))
        assert three[i, j].view(np.uint32) == want.view(np.uint32)
    # only tile (1, 2) is cut, at k = 40: checked against a direct evaluation
    offs = np.zeros(tiles + 1, np.int32)
    offs[1 * 3 + 2 + 1:] = 1
    one = orc.sgemm_fma_pieces(0, 0, 1, A, B, M, N, K, bm, bn, offs, np.array([40], np.int32)).reshape(M, N)
    ref = none.reshape(M, N).copy()
    a2, b2 = A.reshape(M, K), B.reshape(N, K)  # A row-major, B col-major
    for i in range(32, 64):
        for j in range(64, 80):
            p0 = np.float32(0)
            for k in range(40):
                p0 = np.float32(np.float64(a2[i, k]) * np.float64(b2[j, k]) + np.float64(p0))
            p1 = np.float32(0)
            for k in range(40, K):
                p1 = np.float32(np.float64(a2[i, k]) * np.float64(b2[j, k]) + np.float64(p1))
            ref[i, j] = np.float32(p0 + p1)
    assert np.array_equal(one.view(np.uint32), ref.view(np.uint32))
