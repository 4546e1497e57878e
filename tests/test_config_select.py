"""Tuned-table lookup: the selection rule against the reference's own find_best_config
(fixture tests/golden/ref_config_selection.json), the shipped table, and the generator's checks."""
import json
import os
import sys

import pytest

from common import LAYOUTS

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = os.path.join(HERE, "golden")
sys.path.insert(0, os.path.join(HERE, "..", "rocm_sgemm_b200", "config"))


@pytest.fixture(scope="module")
def fixture():
    with open(os.path.join(GOLDEN, "ref_config_selection.json")) as f:
        return json.load(f)


def test_selection_rule_matches_reference(sgemm, fixture):
    table = fixture["sorted_config_map"]  # rows (m, n, k, la, lb, lc, config_idx), the reference's order
    keys = [r[:6] for r in table]
    for s in fixture["selections"]:
        row = sgemm.select_in_table(keys, s["M"], s["N"], s["K"], s["A"], s["B"], s["C"])
        assert row >= 0
        assert table[row][6] == s["config_idx"], s
        assert fixture["kernel_configs"][str(table[row][6])] == s["nine"]


def test_selection_against_reference_build(sgemm, orc, fixture):
    if not orc.have_ref():
        pytest.skip("oracle/_ref not built")
    table = orc.ref_config_map()
    keys = [r[:6] for r in table]
    import itertools
    sizes = [1, 7, 64, 100, 777, 1024, 1500, 3000, 4096, 5000, 8192, 20000]
    for (m, n, k) in itertools.islice(itertools.product(sizes, repeat=3), 0, None, 7):
        for (la, lb, lc) in LAYOUTS:
            row = sgemm.select_in_table(keys, m, n, k, la, lb, lc)
            idx, _ = orc.ref_find_best_config(m, n, k, la, lb, lc)
            assert table[row][6] == idx, (m, n, k, la, lb, lc)


def test_empty_table(sgemm):
    assert sgemm.select_in_table([], 128, 128, 128, 0, 0, 0) == -1


def test_any_layout_fallback(sgemm):
    # no entry with the asked layout: nearest size over all entries (second pass of the rule)
    keys = [(1024, 1024, 1024, 0, 0, 0), (4096, 4096, 4096, 0, 0, 0)]
    assert sgemm.select_in_table(keys, 3000, 3000, 3000, 1, 1, 1) == 1
    assert sgemm.select_in_table(keys, 1500, 1500, 1500, 1, 0, 1) == 0


def test_shipped_table_is_consistent(sgemm):
    entries = sgemm.table_entries()
    assert entries == sorted(entries, key=lambda e: e[:6])
    nv = sgemm.num_variants()
    for (m, n, k, la, lb, lc, v, s) in entries:
        assert 0 <= v < nv and s >= 0  # split_k 0 = equal K ranges per CTA, summed in order inside the kernel
        # every tabled (variant, layout) pair has both kernels built
        assert sgemm.has_kernel(v, la, lb, lc, True) and sgemm.has_kernel(v, la, lb, lc, False)
        p, vi = sgemm.select_config(m, n, k, lc, la, lb)
        assert vi == v and p.split_k == s
    # any problem in any layout resolves to a kernel that exists
    for (la, lb, lc) in LAYOUTS:
        for (m, n, k) in [(1, 1, 1), (320, 320, 320), (5000, 300, 70000), (16384, 2048, 16384)]:
            p, vi = sgemm.select_config(m, n, k, lc, la, lb)
            assert sgemm.has_kernel(vi, la, lb, lc, False)
            assert sgemm.get_gemm_params(m, n, k, lc, la, lb) == p


def test_generator_constraints():
    import generate_config as g
    assert g.check_variant(g.DEFAULT_VARIANT) is None
    bad = list(g.DEFAULT_VARIANT)
    bad[0] = 128  # block_size no longer matches the warp grid
    assert g.check_variant(tuple(bad)) is not None
    bad = list(g.DEFAULT_VARIANT)
    bad[8] = 3  # threads_n must divide 32
    assert g.check_variant(tuple(bad)) is not None
    bad = list(g.DEFAULT_VARIANT)
    bad[3], bad[9] = 64, 8  # 8 stages of 128x128x64: over the shared-memory limit
    assert g.check_variant(tuple(bad)) is not None


def test_generator_output(tmp_path):
    import generate_config as g
    cfg = {"configurations": [
        {"range": {"M": 512, "N": 512, "K": 512}, "layout": {"A": "col_major", "B": "row_major", "C": "row_major"},
         "config": {"block_size": 128, "block_m": 64, "block_n": 128, "block_k": 8, "warp_tile_m_count": 2,
                    "warp_tile_n_count": 2, "thread_tile_m": 4, "thread_tile_n": 4, "threads_n": 8, "split_k": 2}}]}
    p = tmp_path / "c.json"
    p.write_text(json.dumps(cfg))
    variants, entries, pairs = g.generate(str(p), str(tmp_path / "gen"))
    assert g.DEFAULT_VARIANT in variants and len(variants) == 2
    # (variant index, split_k, pretranspose)
    assert entries == [((512, 512, 512, 1, 0, 0), (variants.index((128, 64, 128, 8, 2, 2, 4, 4, 8, 2, 2, 1, 1, 0)), 2, 0))]
    # the tabled pair plus the default variant in all eight layouts
    assert len(pairs) == 9
    names = (tmp_path / "gen" / "sources.txt").read_text().split()
    assert "kernel_lookup.cu" in names and len(names) == 10
