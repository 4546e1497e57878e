"""The C ABI loads without a GPU, exports every function its header declares, and rejects bad
arguments with status codes (no launches are made here)."""
import ctypes
import os
import re

import rocm_sgemm_b200 as pkg

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions(header):
    text = open(header).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return re.findall(r"\b(b200_\w+)\s*\(", text)


def test_exports_match_header(sgemm):
    names = declared_functions(os.path.join(ROOT, "include", "b200_sgemm.h"))
    assert len(names) >= 13
    lib = sgemm.lib()
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/b200_sgemm.h but not exported"
    # the Python mirror binds exactly the declared surface: nothing declared is left out, nothing extra is bound
    assert set(names) == set(pkg.EXPORTS)


def test_cublas_wrapper_exports(sgemm):
    hdr = os.path.join(ROOT, "include", "b200_cublas_wrapper.h")
    if not os.path.exists(hdr) or not os.path.exists(pkg.CUBLAS_LIB_PATH):
        import pytest
        pytest.skip("comparison wrapper not built")
    lib = ctypes.CDLL(pkg.CUBLAS_LIB_PATH)
    for n in declared_functions(hdr):
        assert hasattr(lib, n)


def test_argument_checks_need_no_device(sgemm):
    l = sgemm.lib()
    # null pointers, zero dimension, bad layout: rejected before any CUDA call
    assert l.b200_sgemm(0, 0, 0, None, None, None, 4, 4, 4, None) == pkg.INVALID_ARGUMENT
    assert l.b200_sgemm(0, 0, 0, 16, 16, 16, 0, 4, 4, None) == pkg.INVALID_ARGUMENT
    assert l.b200_sgemm(2, 0, 0, 16, 16, 16, 4, 4, 4, None) == pkg.INVALID_ARGUMENT
    assert l.b200_sgemm(0, 0, 0, 16, 16, 16, 2 ** 31, 4, 4, None) == pkg.UNSUPPORTED_SIZE
    # leading dimension smaller than the packed extent
    assert l.b200_sgemm_ex(0, 0, 0, 16, 16, 16, 8, 8, 8, 4, 0, 0, -1, 0, None, 0, None) == pkg.INVALID_ARGUMENT
    # variant index out of range
    assert l.b200_sgemm_ex(0, 0, 0, 16, 16, 16, 8, 8, 8, 0, 0, 0, 10 ** 6, 0, None, 0, None) == pkg.INVALID_ARGUMENT
    # split-K asked for without a workspace
    assert l.b200_sgemm_ex(0, 0, 0, 16, 16, 16, 64, 64, 4096, 0, 0, 0, -1, 4, None, 0, None) \
        == pkg.WORKSPACE_TOO_SMALL
    assert sgemm.workspace_bytes(0, 0, 0, 64, 64, 4096, split_k=4) == 4 * 64 * 64 * 4
    assert sgemm.workspace_bytes(0, 0, 0, 64, 64, 4096, split_k=1) == 0
    assert "invalid" in sgemm.status_string(pkg.INVALID_ARGUMENT)
    assert sgemm.status_string(0) == "ok"


def test_params_struct_roundtrip(sgemm):
    p = sgemm.get_variant(0)
    assert p.block_size % 32 == 0 and p.stages >= 2 and len(p.nine()) == 9
    import pytest
    with pytest.raises(pkg.SgemmError):
        sgemm.get_variant(-1)
