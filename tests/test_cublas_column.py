"""The vendor comparison column is held to the reference's bar for its own vendor wrapper.

The reference checks rocblas_wrapper::gemm<TA, TB> on its 13 shapes in the four layouts with a
column-major C against the host GEMM, absolute tolerance 1e-4 (test/rocblas/test.cpp:31-186).  Here
b200_cublas_gemm_layout (cublasSgemm, strict FP32 math mode) is checked the same way through its C ABI for
all eight layouts: the four with a row-major C go through the C^T = B^T A^T mapping, whose transpose flags
are exactly what a wrong number in the comparison column would come from.
"""
import ctypes
import os
import subprocess

import numpy as np
import pytest

from common import LAYOUTS, REFERENCE_TEST_SHAPES, layout_name

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cublas(sgemm):
    import rocm_sgemm_b200 as pkg
    if not os.path.exists(pkg.CUBLAS_LIB_PATH):
        from rocm_sgemm_b200 import build
        build.build_cublas_wrapper()
    lib = ctypes.CDLL(pkg.CUBLAS_LIB_PATH)
    i, vp, sz = ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t
    lib.b200_cublas_gemm_layout.argtypes = [i, i, i, vp, vp, vp, sz, sz, sz, vp]
    lib.b200_cublas_gemm.argtypes = [i, i, vp, vp, vp, sz, sz, sz, vp]
    assert lib.b200_cublas_init() == 1
    yield lib
    lib.b200_cublas_cleanup()


@pytest.mark.parametrize("layout", LAYOUTS, ids=lambda l: layout_name(*l))
@pytest.mark.parametrize("shape", REFERENCE_TEST_SHAPES + [(130, 70, 33)], ids=lambda s: "x".join(map(str, s)))
def test_cublas_column_matches_host_gemm(cublas, orc, shape, layout):
    (M, N, K), (la, lb, lc) = shape, layout
    A, B = orc.init_matrix(la, M, K), orc.init_matrix(lb, K, N)
    dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    dC = torch.full((M * N,), float("nan"), dtype=torch.float32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    assert cublas.b200_cublas_gemm_layout(lc, la, lb, dC.data_ptr(), dA.data_ptr(), dB.data_ptr(), M, N, K, stream) == 0
    torch.cuda.synchronize()
    ref = orc.sgemm_f32(lc, la, lb, A, B, M, N, K, threads=orc.max_threads())
    assert np.max(np.abs(dC.cpu().numpy() - ref)) <= 1e-4  # the reference suite's tolerance


@pytest.mark.parametrize("ta,tb", [(0, 0), (1, 0), (0, 1), (1, 1)])
def test_cublas_transpose_entry(cublas, orc, ta, tb):
    """b200_cublas_gemm(transpose_a, transpose_b): the reference wrapper's own signature, column-major C."""
    M, N, K = 320, 512, 192
    la, lb = (0 if ta else 1), (0 if tb else 1)  # a transposed column-major operand is a row-major one
    A, B = orc.init_matrix(la, M, K), orc.init_matrix(lb, K, N)
    dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    dC = torch.full((M * N,), float("nan"), dtype=torch.float32, device="cuda")
    assert cublas.b200_cublas_gemm(ta, tb, dC.data_ptr(), dA.data_ptr(), dB.data_ptr(), M, N, K,
                                   torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    ref = orc.sgemm_f32(1, la, lb, A, B, M, N, K, threads=orc.max_threads())
    assert np.max(np.abs(dC.cpu().numpy() - ref)) <= 1e-4


def test_cublas_test_and_bench_binaries():
    """cublas_test = the CublasTest group of the C++ harness alone; cublas_bench = the vendor rows alone."""
    import json
    bindir = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "rocm_sgemm_b200", "bin")
    if not os.path.exists(os.path.join(bindir, "cublas_test")):
        from rocm_sgemm_b200 import build
        build.build_all()
    r = subprocess.run([os.path.join(bindir, "cublas_test")], capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-1000:]
    assert r.stdout.strip().splitlines()[-1] == "104 tests, 0 failed" and "GEMMTest" not in r.stdout
    r = subprocess.run([os.path.join(bindir, "cublas_bench"), "--json", "--shapes", "512", "--layouts", "rrr,ccc",
                        "--iters", "3", "--warmup", "1"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-1000:]
    rows = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    assert [x["layout"] for x in rows] == ["rrr", "ccc"] and all(x["cublas_avg_tflops"] > 0 for x in rows)
