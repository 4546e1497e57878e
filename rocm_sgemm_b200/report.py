"""Markdown performance report from gemm_bench rows.

Counterpart of the reference's docs/generate_report.py:171-253 (the table of docs/square.md:7-8): one
line per (matrix size, input layout (A,B)) with this library's TFLOP/s for column-major C, the vendor
BLAS for column-major C, their ratio, this library for row-major C and its ratio against the same
vendor figure.  A second table gives the share of the FP32 FMA peak.  Plots are left out (no
matplotlib in the image).

    rocm_sgemm_b200/bin/gemm_bench --json --shapes 1024:2048:4096:8192 > rows.jsonl     # on a B200
    python -m rocm_sgemm_b200.report rows.jsonl --title "Square matrices" --output square.md
    python -m rocm_sgemm_b200.report --run --shapes 1024:2048 --output square.md       # runs gemm_bench itself
"""
from __future__ import annotations

import argparse
import json
import subprocess
import sys
from collections import defaultdict
from pathlib import Path

PKG = Path(__file__).resolve().parent
LAYOUT_ORDER = [("c", "c"), ("r", "c"), ("c", "r"), ("r", "r")]  # the reference's row order


def parse_rows(text: str):
    """gemm_bench --json prints one object per line; anything else (banner, errors) is skipped."""
    rows = []
    for line in text.splitlines():
        line = line.strip()
        if not line.startswith("{"):
            continue
        try:
            r = json.loads(line)
        except json.JSONDecodeError:
            continue
        if {"M", "N", "K", "layout", "avg_tflops"} <= r.keys():
            rows.append(r)
    return rows


def run_gemm_bench(shapes: str, iters: int, warmup: int, exe: Path | None = None, tf32x3: bool = False) -> str:
    exe = exe or PKG / "bin" / "gemm_bench"
    if not exe.exists():
        raise RuntimeError(f"{exe} is missing: run python -m rocm_sgemm_b200.build first")
    cmd = [str(exe), "--json", "--shapes", shapes, "--iters", str(iters), "--warmup", str(warmup)]
    if tf32x3:
        cmd.append("--tf32x3")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=1800)
    if r.returncode != 0:
        raise RuntimeError(f"gemm_bench failed ({r.returncode}): {r.stderr[-2000:]}")
    return r.stdout


def _fmt(x, spec):
    return format(x, spec) if x else "-"


def markdown(rows, title: str, system: str = "", peak_tflops: float | None = None) -> str:
    ours = defaultdict(dict)    # (M,N,K) -> {(la,lb,lc): tflops}
    vendor = defaultdict(dict)
    pct = defaultdict(dict)
    for r in rows:
        size = (r["M"], r["N"], r["K"])
        la, lb, lc = r["layout"][0], r["layout"][1], r["layout"][2]
        ours[size][(la, lb, lc)] = r["avg_tflops"]
        pct[size][(la, lb, lc)] = r.get("pct_fp32_peak")
        if r.get("cublas_avg_tflops"):
            vendor[size][(la, lb, lc)] = r["cublas_avg_tflops"]
    out = [f"# {title}", ""]
    out.append(f"Performance measured on {system} in TFLOPs." if system else "Performance measured in TFLOPs.")
    out += ["", "## FP32 SGEMM Performance Results", ""]
    out.append("| Matrix Size | Input Layout (A,B) | `b200_sgemm`<br>(C=col) | `cuBLAS`<br>(C=col) | Ratio<br>(C=col / cuBLAS) "
               "| `b200_sgemm`<br>(C=row) | Ratio<br>(C=row / cuBLAS) |")
    out.append("|:---|:---|---:|---:|---:|---:|---:|")
    for size in sorted(ours):
        name = "x".join(str(d) for d in size)
        for la, lb in LAYOUT_ORDER:
            col = ours[size].get((la, lb, "c"))
            row = ours[size].get((la, lb, "r"))
            ven = vendor[size].get((la, lb, "c"))
            if col is None and row is None:
                continue
            ratio_c = col / ven if col and ven else None
            ratio_r = row / ven if row and ven else None
            out.append(f"| {name} | ({la},{lb}) | {_fmt(col, '.2f')} | {_fmt(ven, '.2f')} | {_fmt(ratio_c, '.3f')} "
                       f"| {_fmt(row, '.2f')} | {_fmt(ratio_r, '.3f')} |")
    out += ["", "## Share of the FP32 FMA peak" + (f" ({peak_tflops:.2f} TFLOP/s)" if peak_tflops else ""), ""]
    out.append("| Matrix Size | Input Layout (A,B) | C=col % | C=row % |")
    out.append("|:---|:---|---:|---:|")
    for size in sorted(ours):
        name = "x".join(str(d) for d in size)
        for la, lb in LAYOUT_ORDER:
            pc, pr = pct[size].get((la, lb, "c")), pct[size].get((la, lb, "r"))
            if pc is None and pr is None:
                continue
            out.append(f"| {name} | ({la},{lb}) | {_fmt(pc, '.1f')} | {_fmt(pr, '.1f')} |")
    tensor = defaultdict(dict)
    for r in rows:
        if r.get("tf32x3_avg_tflops"):
            tensor[(r["M"], r["N"], r["K"])][tuple(r["layout"])] = r["tf32x3_avg_tflops"]
    if tensor:
        out += ["", "## Optional 3xTF32 tensor-core column (`b200_sgemm_3xtf32`, not the FP32 FMA arithmetic)", ""]
        out.append("| Matrix Size | Input Layout (A,B) | C=col | C=row | C=row / `b200_sgemm` |")
        out.append("|:---|:---|---:|---:|---:|")
        for size in sorted(tensor):
            name = "x".join(str(d) for d in size)
            for la, lb in LAYOUT_ORDER:
                tc, tr = tensor[size].get((la, lb, "c")), tensor[size].get((la, lb, "r"))
                if tc is None and tr is None:
                    continue
                base = ours[size].get((la, lb, "r"))
                out.append(f"| {name} | ({la},{lb}) | {_fmt(tc, '.2f')} | {_fmt(tr, '.2f')} "
                           f"| {_fmt(tr / base if tr and base else None, '.2f')} |")
    return "\n".join(out) + "\n"


def main(argv=None):
    ap = argparse.ArgumentParser(description="markdown report from gemm_bench --json rows")
    ap.add_argument("rows", nargs="?", help="file with gemm_bench --json output ('-' = stdin)")
    ap.add_argument("--run", action="store_true", help="run bin/gemm_bench instead of reading a file")
    ap.add_argument("--shapes", default="1024:2048:4096:8192")
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--tf32x3", action="store_true", help="with --run: also time the optional 3xTF32 entry")
    ap.add_argument("--title", default="Square matrices")
    ap.add_argument("--system", default="NVIDIA B200 (sm_100a), CUDA 12.9")
    ap.add_argument("--peak", type=float, default=74.45, help="FP32 FMA peak in TFLOP/s quoted in the second table")
    ap.add_argument("--note", default="", help="text inserted under the title ('\\n' for line breaks)")
    ap.add_argument("--output", default="-")
    a = ap.parse_args(argv)
    if a.run:
        text = run_gemm_bench(a.shapes, a.iters, a.warmup, tf32x3=a.tf32x3)
    elif a.rows in (None, "-"):
        text = sys.stdin.read()
    else:
        text = Path(a.rows).read_text()
    rows = parse_rows(text)
    if not rows:
        raise SystemExit("no gemm_bench rows found")
    md = markdown(rows, a.title, a.system, a.peak)
    if a.note:  # free text (for instance the commands that produced the rows) placed under the title
        head, rest = md.split("\n", 1)
        md = head + "\n\n" + a.note.replace("\\n", "\n") + "\n" + rest
    if a.output == "-":
        sys.stdout.write(md)
    else:
        Path(a.output).write_text(md)
        print(f"report written to {a.output} ({len(rows)} rows)")


if __name__ == "__main__":
    main()
