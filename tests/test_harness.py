"""The C++ harnesses over the drop-in header (include/rocm_sgemm/gemm.hpp): gemm_test is the reference's
test/gemm/test.cpp suite (13 shapes x 8 layouts, tolerance 1e-4) plus identity and vendor-wrapper cases,
gemm_bench its benchmark/gemm/bench.cpp with the cuBLAS column.  Run as child processes on the GPU box."""
import json
import os
import subprocess

import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

BIN = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "rocm_sgemm_b200", "bin")


def _exe(name):
    path = os.path.join(BIN, name)
    if not os.path.exists(path):
        from rocm_sgemm_b200 import build
        build.build_all()
    return path


def test_gemm_test_suite():
    r = subprocess.run([_exe("gemm_test")], capture_output=True, text=True, timeout=900)
    tail = r.stdout.strip().splitlines()[-1]
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-1000:]
    assert tail.endswith(" 0 failed") and "FAILED" not in r.stdout
    assert "BlasWrapperTest/TT" in r.stdout and "IdentityBitExact512" in r.stdout
    assert r.stdout.count("] CublasTest/") == 104  # the vendor column: 13 shapes x 8 layouts


def test_gemm_bench_rows():
    r = subprocess.run([_exe("gemm_bench"), "--json", "--tf32x3", "--identity", "--shapes", "512", "--layouts", "rrr,crc",
                        "--iters", "3", "--warmup", "1"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-1000:]
    rows = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    assert [x["layout"] for x in rows] == ["rrr", "crc"]
    for x in rows:
        assert x["identity_exact"] is True
        assert x["avg_tflops"] > 0 and x["cublas_avg_tflops"] > 0 and x["tf32x3_avg_tflops"] > 0
    # --batch_count: every matrix of the batch is computed (the timed call is b200_sgemm_strided_batched)
    r = subprocess.run([_exe("gemm_bench"), "--json", "--shapes", "512", "--layouts", "rrr", "--batch_count", "3",
                        "--iters", "3", "--warmup", "1"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-1000:]
    one = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(one) == 1 and one[0]["avg_tflops"] > 0 and one[0]["avg_ms"] > rows[0]["avg_ms"]
