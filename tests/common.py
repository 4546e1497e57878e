"""Shared shapes and helpers of the parity tests."""
import hashlib

import numpy as np

LAYOUTS = [(a, b, c) for a in (0, 1) for b in (0, 1) for c in (0, 1)]  # (layout_A, layout_B, layout_C)

# the reference suite's 13 shapes (test/gemm/test.cpp:113-176)
REFERENCE_TEST_SHAPES = [(128, 128, 128), (128, 256, 128), (128, 128, 256), (256, 128, 128), (256, 256, 256),
                         (320, 320, 320), (320, 512, 512), (512, 320, 320), (512, 512, 320), (512, 320, 512),
                         (512, 512, 512), (1024, 256, 256), (256, 1024, 256)]

# the rectangular / skinny sweep of the benchmark configuration
SWEEP_SHAPES = [(8192, 8192, 1024), (1024, 1024, 16384), (16384, 256, 4096), (256, 16384, 4096), (2048, 6144, 2048),
                (6144, 2048, 8192)]


def layout_name(la, lb, lc):
    return "".join("rc"[x] for x in (la, lb, lc))


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def bits(a: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(a).view(np.uint32)


def as2d(flat: np.ndarray, layout: int, rows: int, cols: int) -> np.ndarray:
    """Logical (rows x cols) view of a packed matrix."""
    return flat.reshape(rows, cols) if layout == 0 else flat.reshape(cols, rows).T


def oracle_chain(sgemm, orc, la, lb, lc, A, B, M, N, K, sm_count, rows=None, variant=-1, split_k=0):
    """The oracle's restatement of what the library computes for this call: one FMA chain per element, or the
    ordered sum of the chains of equal K slices (split-K), or of the tile-dependent K ranges the library reports
    for a device with `sm_count` SMs."""
    blk, offs, bnd = sgemm.stream_plan(lc, la, lb, M, N, K, variant, split_k, sm_count)
    if offs is not None:
        return orc.sgemm_fma_pieces(lc, la, lb, A, B, M, N, K, blk[0], blk[1], offs, bnd, rows=rows,
                                    threads=orc.max_threads())
    p, _ = sgemm.select_config(M, N, K, lc, la, lb)
    if variant >= 0:
        p = sgemm.get_variant(variant)
    s = split_k if split_k > 0 else (p.split_k if variant < 0 else 1)
    return orc.sgemm_fma(lc, la, lb, A, B, M, N, K, rows=rows, splits=max(s, 1), k_align=p.block_k,
                         threads=orc.max_threads())
