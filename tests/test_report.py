"""The markdown report (counterpart of the reference's docs/generate_report.py:171-253) on canned rows."""
import json

from rocm_sgemm_b200 import report


def _row(m, layout, ours, vendor):
    return json.dumps({"name": "x", "M": m, "N": m, "K": m, "layout": layout, "avg_ms": 1.0, "min_ms": 1.0, "max_ms": 1.0,
                       "avg_tflops": ours, "min_time_tflops": ours, "pct_fp32_peak": 100.0 * ours / 74.45,
                       "bytes_per_second": 1e9, "cublas_avg_tflops": vendor, "cublas_min_ms": 1.0, "identity_exact": None})


def test_parse_skips_noise():
    text = "device: something\n" + _row(1024, "rrc", 40.0, 38.0) + "\n{broken\n\n" + _row(1024, "rrr", 41.0, 39.0)
    rows = report.parse_rows(text)
    assert [r["layout"] for r in rows] == ["rrc", "rrr"]


def test_table_rows_and_ratios():
    text = "\n".join(_row(m, la + lb + lc, 60.0 + i, 50.0) for m in (2048, 1024)
                     for i, (la, lb, lc) in enumerate((a, b, c) for a in "rc" for b in "rc" for c in "rc"))
    md = report.markdown(report.parse_rows(text), "Square matrices", "B200", 74.45)
    lines = [l for l in md.splitlines() if l.startswith("| 1024x1024x1024")]
    assert len(lines) == 8  # four (A,B) rows in each of the two tables
    # sizes ascend, (A,B) in the reference's order (c,c) (r,c) (c,r) (r,r)
    first = lines[:4]
    assert [l.split("|")[2].strip() for l in first] == ["(c,c)", "(r,c)", "(c,r)", "(r,r)"]
    # (r,r): ours C=col is layout rrc = index 1 -> 61.0; vendor 50 -> ratio 1.220; C=row rrr = index 0 -> 60.0 -> 1.200
    rr = [l for l in lines if "(r,r)" in l][0].split("|")
    assert [c.strip() for c in rr[3:8]] == ["61.00", "50.00", "1.220", "60.00", "1.200"]
    assert md.index("1024x1024x1024") < md.index("2048x2048x2048")


def test_missing_vendor_column():
    rows = report.parse_rows(_row(512, "ccc", 10.0, 0.0))
    md = report.markdown(rows, "t")
    line = [l for l in md.splitlines() if l.startswith("| 512x512x512")][0]
    assert "| 10.00 | - | - | - | - |" in line


def test_cli_roundtrip(tmp_path):
    src = tmp_path / "rows.jsonl"
    src.write_text(_row(256, "rrr", 5.0, 4.0) + "\n")
    out = tmp_path / "r.md"
    report.main([str(src), "--output", str(out), "--title", "T"])
    assert out.read_text().startswith("# T\n")


def test_tensor_core_column_is_a_separate_table():
    base = json.loads(_row(4096, "rcr", 64.0, 57.0))
    base["tf32x3_avg_tflops"] = 224.0
    md = report.markdown(report.parse_rows(json.dumps(base)), "t")
    assert "## Optional 3xTF32 tensor-core column" in md
    line = [l for l in md.splitlines() if l.startswith("| 4096x4096x4096 | (r,c) | - | 224.00")][0]
    assert line.endswith("| 3.50 |")
    # rows without the key leave the report as it was
    assert "3xTF32" not in report.markdown(report.parse_rows(_row(4096, "rcr", 64.0, 57.0)), "t")
