#!/usr/bin/env python3
"""Regenerates the committed fixtures in this directory from the REFERENCE's own host code.

Needs the reference tree (it is compiled from where it lies into oracle/_ref/ by oracle/Makefile:
init_matrix and sgemm_cpu of test/test.hpp, and the header that
rocm_sgemm/config/generate_config.py emits from the shipped gemm_config.json).  Run from the
repository root:

    make -C oracle REFERENCE_ROOT=/path/to/rocm_sgemm
    python tests/golden/make_golden.py

Outputs
  ref_gemm_small.npz      inputs from the reference's init_matrix (mt19937(1), U(-1,1)) and the output of
                          the reference's sgemm_cpu for one small shape in all eight layout permutations
  ref_gemm_digests.json   SHA-256 of the reference's init_matrix / sgemm_cpu results at shapes its test
                          suite uses (test/gemm/test.cpp:113-176)
  ref_config_selection.json  the reference's sorted_config_map and what its find_best_config picks for the
                          benchmark shapes and the test-suite shapes in every layout
"""
import hashlib
import json
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
import oracle  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
LAYOUTS = [(a, b, c) for a in (0, 1) for b in (0, 1) for c in (0, 1)]

TEST_SHAPES = [(128, 128, 128), (128, 256, 128), (128, 128, 256), (256, 128, 128), (256, 256, 256), (320, 320, 320),
               (320, 512, 512), (512, 320, 320), (512, 512, 320), (512, 320, 512), (512, 512, 512), (1024, 256, 256),
               (256, 1024, 256)]
BENCH_SHAPES = [(256, 256, 256), (4096, 4096, 4096), (8192, 8192, 1024), (1024, 1024, 16384), (16384, 256, 4096),
                (256, 16384, 4096), (2048, 6144, 2048), (6144, 2048, 8192), (16384, 16384, 16384),
                (16384, 8192, 16384), (16384, 4096, 16384), (16384, 2048, 16384), (1024, 1024, 1024),
                (2048, 2048, 2048), (8192, 8192, 8192), (100, 3000, 77)]


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def main():
    assert oracle.have_ref(), "build oracle/_ref first (make -C oracle)"

    # 1. one small problem, all layouts, full data
    M, N, K = 24, 20, 28
    small = {}
    for la in (0, 1):
        small[f"A_{la}"] = oracle.ref_init_matrix(la, M, K)
    for lb in (0, 1):
        small[f"B_{lb}"] = oracle.ref_init_matrix(lb, K, N)
    for (la, lb, lc) in LAYOUTS:
        small[f"C_{la}{lb}{lc}"] = oracle.ref_sgemm_cpu(lc, la, lb, small[f"A_{la}"], small[f"B_{lb}"], M, N, K)
    np.savez_compressed(os.path.join(HERE, "ref_gemm_small.npz"), shape=np.array([M, N, K]), **small)

    # 2. digests at the reference's own test shapes
    dig = {"init_matrix": {}, "sgemm_cpu": {}}
    for (rows, cols) in [(128, 128), (320, 512), (1024, 256)]:
        for lay in (0, 1):
            dig["init_matrix"][f"{rows}x{cols}_{lay}"] = sha(oracle.ref_init_matrix(lay, rows, cols))
    for (m, n, k) in [(128, 128, 128), (128, 256, 128), (320, 320, 320), (256, 1024, 256)]:
        for (la, lb, lc) in LAYOUTS:
            A, B = oracle.ref_init_matrix(la, m, k), oracle.ref_init_matrix(lb, k, n)
            dig["sgemm_cpu"][f"{m}x{n}x{k}_{la}{lb}{lc}"] = sha(oracle.ref_sgemm_cpu(lc, la, lb, A, B, m, n, k))
    with open(os.path.join(HERE, "ref_gemm_digests.json"), "w") as f:
        json.dump(dig, f, indent=1, sort_keys=True)

    # 3. configuration selection
    table = oracle.ref_config_map()  # (m, n, k, la, lb, lc, config_idx)
    sel = []
    for (m, n, k) in TEST_SHAPES + BENCH_SHAPES:
        for (la, lb, lc) in LAYOUTS:
            idx, nine = oracle.ref_find_best_config(m, n, k, la, lb, lc)
            sel.append({"M": m, "N": n, "K": k, "A": la, "B": lb, "C": lc, "config_idx": idx, "nine": list(nine)})
    nines = {}
    for row in table:
        l = oracle.ref_config_lib()
        import ctypes
        out = (ctypes.c_int * 9)()
        l.ref_kernel_config(row[6], out)
        nines[row[6]] = list(out)
    with open(os.path.join(HERE, "ref_config_selection.json"), "w") as f:
        json.dump({"sorted_config_map": [list(r) for r in table],
                   "kernel_configs": {str(k): v for k, v in sorted(nines.items())},
                   "selections": sel}, f, indent=None, separators=(",", ":"))
    print("fixtures written to", HERE)


if __name__ == "__main__":
    main()
