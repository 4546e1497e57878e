"""ctypes front end of the CPU oracle (oracle/sgemm_oracle.c) and, when it has been built, of
the reference's own host code compiled into oracle/_ref/.

Test infrastructure only: imported by tests/, by the smoke check and by the CPU-baseline /
reference arm of the benchmark; never by the product package.

Layouts are 0 = row-major, 1 = col-major; matrices are packed 1-D float32 numpy arrays.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle_sgemm.so")
_REF_GEMM_PATH = os.path.join(_HERE, "_ref", "libref_sgemm.so")
_REF_CFG_PATH = os.path.join(_HERE, "_ref", "libref_config.so")

ROW, COL = 0, 1
_sz = ctypes.c_size_t
_fp = ctypes.POINTER(ctypes.c_float)
_dp = ctypes.POINTER(ctypes.c_double)


def build(reference_root: str | None = None) -> None:
    """Compile the oracle (and oracle/_ref when the reference tree is present) with make."""
    cmd = ["make", "-s", "-C", _HERE]
    if reference_root:
        cmd.append(f"REFERENCE_ROOT={reference_root}")
    subprocess.run(cmd, check=True)


def _load():
    if not os.path.exists(_LIB_PATH):
        build()
    lib = ctypes.CDLL(_LIB_PATH)
    lib.oracle_init_matrix.argtypes = [ctypes.c_int, _sz, _sz, _fp]
    lib.oracle_fill_ab.argtypes = [ctypes.c_uint32, ctypes.c_int, ctypes.c_int, _sz, _sz, _sz, _fp, _fp]
    lib.oracle_fill_pattern.argtypes = [ctypes.c_int, _sz, _sz, _fp]
    lib.oracle_fill_identity.argtypes = [ctypes.c_int, _sz, _sz, _fp]
    lib.oracle_sgemm_f32.argtypes = [ctypes.c_int] * 3 + [_fp, _fp, _fp, _sz, _sz, _sz, _sz, _sz, ctypes.c_int]
    lib.oracle_sgemm_fma.argtypes = [ctypes.c_int] * 3 + [_fp, _fp, _fp, _sz, _sz, _sz, _sz, _sz, ctypes.c_int, _sz,
                                                           ctypes.c_int]
    lib.oracle_sgemm_fma_pieces.argtypes = [ctypes.c_int] * 3 + [_fp, _fp, _fp, _sz, _sz, _sz, _sz, _sz, _sz, _sz,
                                                                  ctypes.POINTER(ctypes.c_int),
                                                                  ctypes.POINTER(ctypes.c_int), ctypes.c_int]
    lib.oracle_sgemm_f64.argtypes = [ctypes.c_int] * 3 + [_dp, _fp, _fp, _sz, _sz, _sz, _sz, _sz, ctypes.c_int]
    lib.oracle_error_metrics.argtypes = [ctypes.c_int, _fp, _dp, _sz, _sz, _sz, _sz, _dp]
    lib.oracle_max_threads.restype = ctypes.c_int
    return lib


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = _load()
    return _lib


def _f(a: np.ndarray):
    assert a.dtype == np.float32 and a.flags.c_contiguous
    return a.ctypes.data_as(_fp)


def _d(a: np.ndarray):
    assert a.dtype == np.float64 and a.flags.c_contiguous
    return a.ctypes.data_as(_dp)


def max_threads() -> int:
    return int(lib().oracle_max_threads())


def init_matrix(layout: int, rows: int, cols: int) -> np.ndarray:
    """The reference test's init_matrix: mt19937(1), U(-1,1), logical order (test/test.hpp:11-25)."""
    out = np.empty(rows * cols, dtype=np.float32)
    lib().oracle_init_matrix(layout, rows, cols, _f(out))
    return out


def fill_ab(seed: int, la: int, lb: int, M: int, N: int, K: int, with_b: bool = True):
    """A (MxK) then B (KxN) from ONE mt19937(seed) stream of U(-1,1), logical order."""
    A = np.empty(M * K, dtype=np.float32)
    B = np.empty(K * N, dtype=np.float32) if with_b else None
    lib().oracle_fill_ab(seed, la, lb, M, N, K, _f(A), _f(B) if with_b else None)
    return A, B


def fill_pattern(layout: int, rows: int, cols: int) -> np.ndarray:
    out = np.empty(rows * cols, dtype=np.float32)
    lib().oracle_fill_pattern(layout, rows, cols, _f(out))
    return out


def fill_identity(layout: int, rows: int, cols: int) -> np.ndarray:
    out = np.empty(rows * cols, dtype=np.float32)
    lib().oracle_fill_identity(layout, rows, cols, _f(out))
    return out


def _band(M, rows):
    r0, r1 = (0, M) if rows is None else rows
    assert 0 <= r0 <= r1 <= M
    return r0, r1


def sgemm_f32(lc, la, lb, A, B, M, N, K, rows=None, threads=1, out=None) -> np.ndarray:
    """sgemm_cpu restated (test/test.hpp:30-45): float accumulator, k ascending, mul then add."""
    C = np.zeros(M * N, dtype=np.float32) if out is None else out
    r0, r1 = _band(M, rows)
    lib().oracle_sgemm_f32(lc, la, lb, _f(C), _f(A), _f(B), M, N, K, r0, r1, threads)
    return C


def sgemm_fma(lc, la, lb, A, B, M, N, K, rows=None, splits=1, k_align=1, threads=1) -> np.ndarray:
    """k-ascending fused-multiply-add chain(s): the arithmetic the GPU kernels perform."""
    C = np.zeros(M * N, dtype=np.float32)
    r0, r1 = _band(M, rows)
    lib().oracle_sgemm_fma(lc, la, lb, _f(C), _f(A), _f(B), M, N, K, r0, r1, splits, k_align, threads)
    return C


def sgemm_fma_pieces(lc, la, lb, A, B, M, N, K, block_m, block_n, offsets, bounds, rows=None, threads=1) -> np.ndarray:
    """FMA chains with per-tile K cut points: the last piece's chain plus the earlier pieces in ascending K order (offsets / bounds as returned by the
    library's stream_plan: offsets has tiles + 1 entries, tile = tile_row * ceil(N / block_n) + tile_column)."""
    C = np.zeros(M * N, dtype=np.float32)
    r0, r1 = _band(M, rows)
    offs = np.ascontiguousarray(offsets, dtype=np.int32)
    bnd = np.ascontiguousarray(bounds if len(bounds) else [0], dtype=np.int32)
    ip = ctypes.POINTER(ctypes.c_int)
    lib().oracle_sgemm_fma_pieces(lc, la, lb, _f(C), _f(A), _f(B), M, N, K, r0, r1, block_m, block_n,
                                  offs.ctypes.data_as(ip), bnd.ctypes.data_as(ip), threads)
    return C


def sgemm_f64(lc, la, lb, A, B, M, N, K, rows=None, threads=1) -> np.ndarray:
    C = np.zeros(M * N, dtype=np.float64)
    r0, r1 = _band(M, rows)
    lib().oracle_sgemm_f64(lc, la, lb, _d(C), _f(A), _f(B), M, N, K, r0, r1, threads)
    return C


def error_metrics(lc, C, ref64, M, N, rows=None) -> dict:
    """max_abs, max_rel (= |c-ref| / max(|ref|, rms(ref))), rms(ref) and rms(c-ref) over the row band."""
    out = np.zeros(4, dtype=np.float64)
    r0, r1 = _band(M, rows)
    lib().oracle_error_metrics(lc, _f(C), _d(ref64), M, N, r0, r1, _d(out))
    return {"max_abs": float(out[0]), "max_rel": float(out[1]), "rms_ref": float(out[2]),
            "rms_err": float(out[3])}


# --------------------------------------------------------------------------------------------
# the reference's own host code (oracle/_ref), when built
# --------------------------------------------------------------------------------------------
def have_ref() -> bool:
    return os.path.exists(_REF_GEMM_PATH) and os.path.exists(_REF_CFG_PATH)


_ref_gemm = None
_ref_cfg = None


def ref_gemm_lib():
    global _ref_gemm
    if _ref_gemm is None:
        l = ctypes.CDLL(_REF_GEMM_PATH)
        l.ref_init_matrix.argtypes = [ctypes.c_int, _sz, _sz, _fp]
        l.ref_sgemm_cpu.argtypes = [ctypes.c_int] * 3 + [_fp, _fp, _fp, _sz, _sz, _sz]
        _ref_gemm = l
    return _ref_gemm


def ref_init_matrix(layout, rows, cols) -> np.ndarray:
    out = np.empty(rows * cols, dtype=np.float32)
    ref_gemm_lib().ref_init_matrix(layout, rows, cols, _f(out))
    return out


def ref_sgemm_cpu(lc, la, lb, A, B, M, N, K) -> np.ndarray:
    C = np.zeros(M * N, dtype=np.float32)
    ref_gemm_lib().ref_sgemm_cpu(lc, la, lb, _f(C), _f(A), _f(B), M, N, K)
    return C


def ref_config_lib():
    global _ref_cfg
    if _ref_cfg is None:
        l = ctypes.CDLL(_REF_CFG_PATH)
        l.ref_find_best_config.argtypes = [_sz, _sz, _sz, ctypes.c_int, ctypes.c_int, ctypes.c_int]
        l.ref_kernel_config.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_int)]
        l.ref_map_entry.argtypes = [ctypes.c_int, ctypes.POINTER(_sz)]
        _ref_cfg = l
    return _ref_cfg


def ref_find_best_config(M, N, K, la, lb, lc) -> tuple:
    """The reference's selected nine-integer configuration for (M,N,K,layout_A,layout_B,layout_C)."""
    l = ref_config_lib()
    idx = l.ref_find_best_config(M, N, K, la, lb, lc)
    out = (ctypes.c_int * 9)()
    l.ref_kernel_config(idx, out)
    return idx, tuple(out)


def ref_config_map() -> list:
    l = ref_config_lib()
    res = []
    for i in range(l.ref_map_entries()):
        out = (_sz * 7)()
        l.ref_map_entry(i, out)
        res.append(tuple(int(x) for x in out))
    return res
