"""rocm_sgemm_b200 — Python front end of the B200 FP32 GEMM library.

A thin ctypes binding of the C ABI in include/b200_sgemm.h that mirrors the reference's operator
surface: `gemm(layout_C, layout_A, layout_B, C, A, B, M, N, K, stream)` for
rocm_sgemm::gemm<layout_C, layout_A, layout_B>(C, A, B, M, N, K, stream)
(rocm_sgemm/include/rocm_sgemm/gemm.hpp:51-52) and `get_gemm_params` for
rocm_sgemm::get_gemm_params (rocm_sgemm/config/generate_config.py:282-303).

Device memory is the caller's: arguments are raw device addresses (ints) or objects with a
`data_ptr()` method (torch tensors are used for device memory and streams only).  There is no CPU
path: if the compiled library is missing, importing the compute entry points raises.
"""
from __future__ import annotations

import ctypes
import enum
import os
from dataclasses import dataclass

_HERE = os.path.dirname(os.path.abspath(__file__))
# B200_SGEMM_LIB selects another build of the same ABI (the tuner loads candidate builds this way)
LIB_PATH = os.environ.get("B200_SGEMM_LIB") or os.path.join(_HERE, "libb200_sgemm.so")
CUBLAS_LIB_PATH = os.path.join(_HERE, "libb200_cublas_wrapper.so")


class m_layout(enum.IntEnum):
    """rocm_sgemm::m_layout (rocm_sgemm/include/rocm_sgemm/kernel/common.hpp:36-40)."""
    row_major = 0
    col_major = 1


ROW, COL = m_layout.row_major, m_layout.col_major

OK = 0
INVALID_ARGUMENT = -1
NO_KERNEL = -2
WORKSPACE_TOO_SMALL = -3
UNSUPPORTED_SIZE = -4
SCRATCH_LIMIT = -5
STATIC_SCRATCH_BYTES = 32 * 1024 * 1024


class _Params(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int) for n in (
        "block_size", "block_m", "block_n", "block_k", "warp_tile_m_count", "warp_tile_n_count", "thread_tile_m",
        "thread_tile_n", "threads_n", "stages", "fma_mode", "raster", "min_blocks", "pipeline", "split_k", "pretranspose")]


@dataclass(frozen=True)
class gemm_params:
    """struct gemm_params of the reference's generated header plus the CUDA-side knobs."""
    block_size: int
    block_m: int
    block_n: int
    block_k: int
    warp_tile_m_count: int
    warp_tile_n_count: int
    thread_tile_m: int
    thread_tile_n: int
    threads_n: int
    stages: int
    fma_mode: int
    raster: int
    min_blocks: int
    pipeline: int
    split_k: int
    pretranspose: int

    def nine(self) -> tuple:
        return (self.block_size, self.block_m, self.block_n, self.block_k, self.warp_tile_m_count,
                self.warp_tile_n_count, self.thread_tile_m, self.thread_tile_n, self.threads_n)


class SgemmError(RuntimeError):
    def __init__(self, status: int, what: str):
        super().__init__(f"b200_sgemm: {what} (status {status})")
        self.status = status


_lib = None
_sz = ctypes.c_size_t
_vp = ctypes.c_void_p

EXPORTS = ("b200_sgemm", "b200_sgemm_ex", "b200_sgemm_workspace_bytes", "b200_sgemm_select_config",
           "b200_sgemm_num_variants", "b200_sgemm_get_variant", "b200_sgemm_num_entries", "b200_sgemm_get_entry",
           "b200_sgemm_get_entry_pretranspose", "b200_sgemm_map_tile",
           "b200_sgemm_has_kernel", "b200_sgemm_select_in_table", "b200_sgemm_fma_peak", "b200_sgemm_device_status",
           "b200_sgemm_splitk_static", "b200_sgemm_host", "b200_sgemm_host_submit", "b200_sgemm_host_wait", "b200_sgemm_host_plan",
           "b200_sgemm_host_plan_pipelined", "b200_sgemm_release_stream",
           "b200_sgemm_shutdown_host", "b200_sgemm_shutdown",
           "b200_sgemm_status_string", "b200_sgemm_3xtf32", "b200_sgemm_3xtf32_device_status",
           "b200_sgemm_3xtf32_shutdown", "b200_sgemm_strided_batched", "b200_sgemm_blas",
           "b200_sgemm_blas_shutdown", "b200_sgemm_multi", "b200_sgemm_stream_plan",
           "b200_sgemm_selftest_bounded_wait", "b200_sgemm_trial")


def lib() -> ctypes.CDLL:
    """Load libb200_sgemm.so; raises if it has not been built (there is no fallback)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: build it with `python -m rocm_sgemm_b200.build` "
                          "(the library has no CPU or PyTorch fallback)")
    l = ctypes.CDLL(LIB_PATH)
    i = ctypes.c_int
    l.b200_sgemm.argtypes = [i, i, i, _vp, _vp, _vp, _sz, _sz, _sz, _vp]
    l.b200_sgemm_ex.argtypes = [i, i, i, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _sz, _sz, i, i, _vp, _sz, _vp]
    l.b200_sgemm_workspace_bytes.argtypes = [i, i, i, _sz, _sz, _sz, i, i]
    l.b200_sgemm_workspace_bytes.restype = _sz
    l.b200_sgemm_select_config.argtypes = [i, i, i, _sz, _sz, _sz, ctypes.POINTER(_Params), ctypes.POINTER(i)]
    l.b200_sgemm_get_variant.argtypes = [i, ctypes.POINTER(_Params)]
    l.b200_sgemm_get_entry.argtypes = [i, ctypes.POINTER(_sz), ctypes.POINTER(i), ctypes.POINTER(i),
                                       ctypes.POINTER(i)]
    l.b200_sgemm_has_kernel.argtypes = [i, i, i]
    l.b200_sgemm_select_in_table.argtypes = [ctypes.POINTER(_sz), _sz, _sz, _sz, _sz, i, i, i]
    l.b200_sgemm_fma_peak.argtypes = [i, i, ctypes.POINTER(ctypes.c_float), ctypes.POINTER(ctypes.c_double), _vp]
    l.b200_sgemm_device_status.argtypes = [ctypes.POINTER(i)]
    l.b200_sgemm_host.argtypes = [i, i, i, _vp, _vp, _vp, _sz, _sz, _sz]
    l.b200_sgemm_host_submit.argtypes = [i, i, i, _vp, _vp, _vp, _sz, _sz, _sz, ctypes.POINTER(ctypes.c_longlong)]
    l.b200_sgemm_host_wait.argtypes = [ctypes.c_longlong]
    l.b200_sgemm_host_plan.argtypes = [_sz, _sz, _sz, i, ctypes.POINTER(_sz), ctypes.POINTER(i), i]
    l.b200_sgemm_release_stream.argtypes = [ctypes.c_void_p]
    l.b200_sgemm_host_plan_pipelined.argtypes = [_sz, _sz, _sz, i, ctypes.POINTER(_sz), ctypes.POINTER(i), i]
    l.b200_sgemm_splitk_static.argtypes = [i, i, i, _vp, _vp, _vp, _sz, _sz, _sz, i, _vp]
    l.b200_sgemm_3xtf32.argtypes = [i, i, i, _vp, _vp, _vp, _sz, _sz, _sz, _vp]
    l.b200_sgemm_multi.argtypes = [i, i, i, ctypes.POINTER(_vp), i, _vp, _vp, _sz, _sz, _sz, _sz, _sz, _sz, i, _vp]
    l.b200_sgemm_strided_batched.argtypes =[i, i, i, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _sz, _sz, _sz, _vp]
    l.b200_sgemm_blas.argtypes = [i, i, _sz, _sz, _sz, ctypes.c_float, _vp, _sz, _vp, _sz, ctypes.c_float, _vp, _sz, _vp]
    ip = ctypes.POINTER(i)
    l.b200_sgemm_stream_plan.argtypes = [i, i, i, _sz, _sz, _sz, i, i, i, ip, ip, ip, i]
    l.b200_sgemm_selftest_bounded_wait.argtypes = [_vp, _vp, _vp, _vp]
    l.b200_sgemm_trial.argtypes = [i, i, i, _vp, _vp, _vp, _sz, _sz, _sz, i, i, i, _vp]
    l.b200_sgemm_status_string.argtypes = [i]
    l.b200_sgemm_status_string.restype = ctypes.c_char_p
    _lib = l
    return l


def status_string(status: int) -> str:
    return lib().b200_sgemm_status_string(status).decode()


def _check(status: int) -> None:
    if status != 0:
        raise SgemmError(status, status_string(status))


def _ptr(x) -> int:
    if x is None:
        return 0
    if hasattr(x, "data_ptr"):
        return int(x.data_ptr())
    return int(x)


def _stream(stream) -> int:
    """Accepts None (the current torch stream when torch is loaded, else the default stream), a raw
    cudaStream_t value, or an object with a `cuda_stream` attribute (torch.cuda.Stream)."""
    if stream is None:
        try:
            import torch
            if torch.cuda.is_available():
                return int(torch.cuda.current_stream().cuda_stream)
        except ImportError:
            pass
        return 0
    if hasattr(stream, "cuda_stream"):
        return int(stream.cuda_stream)
    return int(stream)


def _to_params(p: _Params) -> gemm_params:
    return gemm_params(*(getattr(p, n) for n, _ in _Params._fields_))


def gemm(layout_c, layout_a, layout_b, C, A, B, M: int, N: int, K: int, stream=None) -> None:
    """C = A @ B on the device, C overwritten; asynchronous on `stream`.  Argument order follows the
    reference: template arguments (layout_C, layout_A, layout_B), then (C, A, B, M, N, K, stream)."""
    _check(lib().b200_sgemm(int(layout_c), int(layout_a), int(layout_b), _ptr(C), _ptr(A), _ptr(B), M, N, K,
                            _stream(stream)))


def gemm_ex(layout_c, layout_a, layout_b, C, A, B, M: int, N: int, K: int, lda: int = 0, ldb: int = 0, ldc: int = 0,
            variant: int = -1, split_k: int = 0, workspace=None, workspace_bytes: int = 0, stream=None) -> None:
    """The explicit form: leading dimensions (0 = packed), forced variant / split-K, caller workspace."""
    _check(lib().b200_sgemm_ex(int(layout_c), int(layout_a), int(layout_b), _ptr(C), _ptr(A), _ptr(B), M, N, K, lda,
                               ldb, ldc, variant, split_k, _ptr(workspace), workspace_bytes, _stream(stream)))


def gemm_trial(layout_c, layout_a, layout_b, C, A, B, M: int, N: int, K: int, variant: int, split_k: int = 1,
               pretranspose: int = 0, stream=None) -> None:
    """What gemm() would do if the table entry of this problem named (variant, split_k, pretranspose)."""
    _check(lib().b200_sgemm_trial(int(layout_c), int(layout_a), int(layout_b), _ptr(C), _ptr(A), _ptr(B), M, N, K, variant,
                                  split_k, pretranspose, _stream(stream)))


def gemm_splitk_static(layout_c, layout_a, layout_b, C, A, B, M: int, N: int, K: int, split_k: int, stream=None) -> None:
    """Split-K GEMM whose partial sums live in the library's built-in 32 MiB device array: for callers
    that may not allocate device memory.  Raises SgemmError(SCRATCH_LIMIT) when split_k*M*N floats do not
    fit.  Calls on one device share the array: do not let two of them overlap on the GPU."""
    _check(lib().b200_sgemm_splitk_static(int(layout_c), int(layout_a), int(layout_b), _ptr(C), _ptr(A), _ptr(B), M,
                                          N, K, split_k, _stream(stream)))


def gemm_host(layout_c, layout_a, layout_b, C, A, B, M: int, N: int, K: int) -> None:
    """C = A @ B for HOST matrices (raw addresses or tensors; page-locked for full speed): uploads, multiplies and
    downloads in one pipelined, blocking call (b200_sgemm_host)."""
    _check(lib().b200_sgemm_host(int(layout_c), int(layout_a), int(layout_b), _ptr(C), _ptr(A), _ptr(B), M, N, K))


def gemm_multi(layout_c, layout_a, layout_b, C_list, A, B, M: int, N: int, K: int, lda: int = 0, ldb: int = 0,
               ldc: int = 0, variant: int = -1, stream=None) -> None:
    """The product stored to every destination in C_list (tensors or raw device addresses, peer mappings included):
    the epilogue of one kernel writes each tile to all of them (b200_sgemm_multi)."""
    ptrs = (_vp * len(C_list))(*[_ptr(c) for c in C_list])
    _check(lib().b200_sgemm_multi(int(layout_c), int(layout_a), int(layout_b), ptrs, len(C_list), _ptr(A), _ptr(B), M, N,
                                  K, lda, ldb, ldc, variant, _stream(stream)))


def gemm_strided_batched(layout_c, layout_a, layout_b, C, A, B, M: int, N: int, K: int, stride_c: int, stride_a: int,
                         stride_b: int, batch: int, stream=None) -> None:
    """`batch` products at fixed element strides (stride_a / stride_b may be 0 to share an operand)."""
    _check(lib().b200_sgemm_strided_batched(int(layout_c), int(layout_a), int(layout_b), _ptr(C), _ptr(A), _ptr(B), M, N,
                                            K, stride_c, stride_a, stride_b, batch, _stream(stream)))


def gemm_blas(trans_a: bool, trans_b: bool, M: int, N: int, K: int, alpha: float, A, lda: int, B, ldb: int, beta: float,
              C, ldc: int, stream=None) -> None:
    """Vendor-BLAS convention: column-major C = alpha * op(A) op(B) + beta * C with leading dimensions."""
    _check(lib().b200_sgemm_blas(int(bool(trans_a)), int(bool(trans_b)), M, N, K, float(alpha), _ptr(A), lda, _ptr(B),
                                 ldb, float(beta), _ptr(C), ldc, _stream(stream)))


def gemm_3xtf32(layout_c, layout_a, layout_b, C, A, B, M: int, N: int, K: int, stream=None) -> None:
    """The optional tensor-core column (b200_sgemm_3xtf32): same arguments as gemm(), FP32 operands split
    into two TF32 halves, three tcgen05 products per pair.  Not bit-identical to gemm()."""
    _check(lib().b200_sgemm_3xtf32(int(layout_c), int(layout_a), int(layout_b), _ptr(C), _ptr(A), _ptr(B), M, N, K,
                                   _stream(stream)))


def tf32x3_device_status() -> int:
    """Synchronises the device; 0 unless a bounded wait inside the 3xTF32 kernel gave up."""
    return int(lib().b200_sgemm_3xtf32_device_status())


def gemm_host_submit(layout_c, layout_a, layout_b, C, A, B, M: int, N: int, K: int) -> int:
    """Enqueues the host-buffer GEMM and returns a ticket at once (b200_sgemm_host_submit).  Up to two jobs are in
    flight per device; the host buffers must stay valid and untouched until gemm_host_wait(ticket) returns."""
    t = ctypes.c_longlong(-1)
    _check(lib().b200_sgemm_host_submit(int(layout_c), int(layout_a), int(layout_b), _ptr(C), _ptr(A), _ptr(B), M, N, K,
                                        ctypes.byref(t)))
    return int(t.value)


def host_plan(M: int, N: int, K: int, sm_count: int = 148, pipelined: bool = False) -> list:
    """Strips of C the host-buffer entries compute, in launch order: [((r0, rows, c0, cols), split_k), ...]; `pipelined`:
    the coarser schedule of a job submitted while another one is in flight."""
    fn = lib().b200_sgemm_host_plan_pipelined if pipelined else lib().b200_sgemm_host_plan
    n = fn(M, N, K, sm_count, None, None, 0)
    if n < 0:
        raise SgemmError(n, status_string(n))
    rects, splits = (_sz * (4 * n))(), (ctypes.c_int * n)()
    fn(M, N, K, sm_count, rects, splits, n)
    return [(tuple(rects[4 * i:4 * i + 4]), splits[i]) for i in range(n)]


def gemm_host_wait(ticket: int) -> None:
    """Blocks until the job behind `ticket` has its C complete in host memory."""
    _check(lib().b200_sgemm_host_wait(int(ticket)))


def stream_plan(layout_c, layout_a, layout_b, M: int, N: int, K: int, variant: int = -1, split_k: int = 0,
                sm_count: int = 148):
    """K cut points of the equal-ranges schedule: ((block_m, block_n, block_k), offsets, bounds) with numpy int32
    arrays (offsets has tiles + 1 entries), or ((block_m, block_n, block_k), None, None) when the call would not use it."""
    import numpy as np
    blk = (ctypes.c_int * 3)()
    n = lib().b200_sgemm_stream_plan(int(layout_c), int(layout_a), int(layout_b), M, N, K, variant, split_k, sm_count,
                                     blk, None, None, 0)
    if n < 0:
        raise SgemmError(n, status_string(n))
    if n == 0:
        return tuple(blk), None, None
    tiles = -(-M // blk[0]) * -(-N // blk[1])
    cap = max(tiles + 1, n)
    offs, bnd = (ctypes.c_int * cap)(), (ctypes.c_int * cap)()
    lib().b200_sgemm_stream_plan(int(layout_c), int(layout_a), int(layout_b), M, N, K, variant, split_k, sm_count, blk,
                                 offs, bnd, cap)
    return tuple(blk), np.array(offs[:tiles + 1], dtype=np.int32), np.array(bnd[:n], dtype=np.int32)


def workspace_bytes(layout_c, layout_a, layout_b, M, N, K, variant: int = -1, split_k: int = 0) -> int:
    return int(lib().b200_sgemm_workspace_bytes(int(layout_c), int(layout_a), int(layout_b), M, N, K, variant,
                                                split_k))


def get_gemm_params(m: int, n: int, k: int, layout_c, layout_a, layout_b) -> gemm_params:
    """rocm_sgemm::get_gemm_params(m, n, k, layout_c, layout_a, layout_b)."""
    return select_config(m, n, k, layout_c, layout_a, layout_b)[0]


def select_config(m, n, k, layout_c, layout_a, layout_b):
    p, v = _Params(), ctypes.c_int(-1)
    _check(lib().b200_sgemm_select_config(int(layout_c), int(layout_a), int(layout_b), m, n, k, ctypes.byref(p),
                                          ctypes.byref(v)))
    return _to_params(p), v.value


def num_variants() -> int:
    return int(lib().b200_sgemm_num_variants())


def get_variant(idx: int) -> gemm_params:
    p = _Params()
    _check(lib().b200_sgemm_get_variant(idx, ctypes.byref(p)))
    return _to_params(p)


def table_entries() -> list:
    """[(M, N, K, layout_A, layout_B, layout_C, variant, split_k), ...] in lookup order."""
    l, out = lib(), []
    for i in range(l.b200_sgemm_num_entries()):
        mnk, lay, v, s = (_sz * 3)(), (ctypes.c_int * 3)(), ctypes.c_int(), ctypes.c_int()
        _check(l.b200_sgemm_get_entry(i, mnk, lay, ctypes.byref(v), ctypes.byref(s)))
        out.append((int(mnk[0]), int(mnk[1]), int(mnk[2]), lay[0], lay[1], lay[2], v.value, s.value))
    return out


def map_tile(raster: int, tile_id: int, grid_m: int, grid_n: int) -> tuple:
    """(tile_m, tile_n) of position `tile_id` in the tile order of a raster mode (0 row, 1 bands, 2 Hilbert)."""
    tm, tn = ctypes.c_int(), ctypes.c_int()
    _check(lib().b200_sgemm_map_tile(raster, tile_id, grid_m, grid_n, ctypes.byref(tm), ctypes.byref(tn)))
    return tm.value, tn.value


def has_kernel(variant: int, layout_a, layout_b, layout_c, aligned: bool) -> bool:
    return bool(lib().b200_sgemm_has_kernel(variant, int(layout_a) * 4 + int(layout_b) * 2 + int(layout_c),
                                            1 if aligned else 0))


def select_in_table(keys, m, n, k, layout_a, layout_b, layout_c) -> int:
    """The selection rule over a caller-supplied sorted table of (m, n, k, la, lb, lc) rows."""
    flat = (_sz * (6 * len(keys)))(*[int(x) for row in keys for x in row])
    return int(lib().b200_sgemm_select_in_table(flat, len(keys), m, n, k, int(layout_a), int(layout_b),
                                                int(layout_c)))


def fma_peak(mode: int = 1, iterations: int = 4096, stream=None) -> dict:
    """Register-only FMA probe: {'ms', 'flops', 'tflops'} for fma.rn.f32 (mode 0) or fma.rn.f32x2 (mode 1)."""
    ms, fl = ctypes.c_float(), ctypes.c_double()
    _check(lib().b200_sgemm_fma_peak(mode, iterations, ctypes.byref(ms), ctypes.byref(fl), _stream(stream)))
    return {"ms": ms.value, "flops": fl.value, "tflops": fl.value / (ms.value * 1e-3) / 1e12}


def selftest_bounded_wait(C, A, B, stream=None) -> None:
    """Launches the one-tile self-test whose consumers run into their (1 ms) wait limit; device_status() then reads
    1 once.  C: 128*128 floats, A: 128*64, B: 64*128 device buffers."""
    _check(lib().b200_sgemm_selftest_bounded_wait(_ptr(C), _ptr(A), _ptr(B), _stream(stream)))


def device_status() -> int:
    """Synchronises the current device and returns (then clears) its kernel status word; 0 = healthy."""
    st = ctypes.c_int(0)
    _check(lib().b200_sgemm_device_status(ctypes.byref(st)))
    return st.value


def release_stream(stream=None) -> None:
    """Frees the drop-in entry's scratch arena of (current device, stream) after synchronising the stream."""
    _check(lib().b200_sgemm_release_stream(_stream(stream)))


def shutdown() -> None:
    _check(lib().b200_sgemm_shutdown())
