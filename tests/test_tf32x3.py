"""The optional tensor-core column b200_sgemm_3xtf32 (tcgen05 / tensor memory, FP32 split into two TF32 halves).

Not the reference's arithmetic, so no bit-exact bar: the result must stay within the float64 bound the
true-FP32 path is held to (max relative error <= 1e-5 * sqrt(K), relative to max(|ref|, rms(ref))), and
well inside it in practice (a few 1e-7 * sqrt(K)); a plain single-TF32 product would miss the tighter
bar by two orders of magnitude, which is what the test of the split checks.
"""
import math

import numpy as np
import pytest

from common import LAYOUTS, layout_name

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def view(t, layout, rows, cols):
    return t.view(rows, cols) if layout == 0 else t.view(cols, rows).T


def rel_err(C2, ref):
    rms = ref.pow(2).mean().sqrt()
    return ((C2.double() - ref).abs() / torch.maximum(ref.abs(), rms)).max().item()


def run(sgemm, la, lb, lc, M, N, K, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    A = torch.rand(M * K, device="cuda", generator=g) * 2 - 1
    B = torch.rand(K * N, device="cuda", generator=g) * 2 - 1
    C = torch.full((M * N,), float("nan"), device="cuda")
    sgemm.gemm_3xtf32(lc, la, lb, C, A, B, M, N, K)
    torch.cuda.synchronize()
    ref = view(A, la, M, K).double() @ view(B, lb, K, N).double()
    return rel_err(view(C, lc, M, N), ref), A, B, C


@pytest.mark.parametrize("layout", LAYOUTS, ids=lambda l: layout_name(*l))
def test_layouts_1024(sgemm, layout):
    la, lb, lc = layout
    M = N = K = 1024
    err, *_ = run(sgemm, la, lb, lc, M, N, K, 21)
    assert err <= 1e-5 * math.sqrt(K), err
    assert err <= 4e-7 * math.sqrt(K), err  # the split recovers FP32-like accuracy (one TF32 product: ~3e-4)
    assert sgemm.tf32x3_device_status() == 0


@pytest.mark.parametrize("shape", [(128, 128, 32), (130, 70, 33), (257, 129, 100), (1000, 200, 36), (64, 300, 520),
                                   (1024, 512, 2048)], ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("layout", [(0, 1, 0), (1, 0, 1), (0, 0, 0)], ids=lambda l: layout_name(*l))
def test_ragged_shapes(sgemm, shape, layout):
    (M, N, K), (la, lb, lc) = shape, layout
    err, *_ = run(sgemm, la, lb, lc, M, N, K, 22)
    assert err <= 4e-7 * math.sqrt(max(K, 64)), err
    assert sgemm.tf32x3_device_status() == 0


def test_full_size_4096(sgemm):
    M = N = K = 4096
    err, A, B, C = run(sgemm, 0, 1, 0, M, N, K, 23)
    assert err <= 4e-7 * math.sqrt(K), err
    # many tiles per CTA: every one of them written (no NaN left from the fill)
    assert not torch.isnan(C).any()
    assert sgemm.tf32x3_device_status() == 0


def test_agrees_with_fp32_path(sgemm):
    """Against the library's own FP32 FMA result: differences of the order of FP32 rounding only."""
    M, N, K = 768, 640, 512
    g = torch.Generator(device="cuda").manual_seed(24)
    A = torch.rand(M * K, device="cuda", generator=g) * 2 - 1
    B = torch.rand(K * N, device="cuda", generator=g) * 2 - 1
    C1 = torch.empty(M * N, device="cuda")
    C2 = torch.empty(M * N, device="cuda")
    sgemm.gemm(0, 0, 0, C1, A, B, M, N, K)
    sgemm.gemm_3xtf32(0, 0, 0, C2, A, B, M, N, K)
    torch.cuda.synchronize()
    assert (C1 - C2).abs().max().item() <= 1e-4  # |c| reaches ~25 here: a few ulp
    assert sgemm.tf32x3_device_status() == 0


def test_argument_errors(sgemm):
    A = torch.zeros(16, device="cuda")
    with pytest.raises(sgemm.SgemmError):
        sgemm.gemm_3xtf32(0, 0, 0, A, A, A, 0, 4, 4)
    with pytest.raises(sgemm.SgemmError):
        sgemm.gemm_3xtf32(0, 0, 2, A, A, A, 4, 4, 4)
    with pytest.raises(sgemm.SgemmError):
        sgemm.gemm_3xtf32(0, 0, 0, None, A, A, 4, 4, 4)


def test_two_streams(sgemm):
    """Calls that repack their operands (col-major A, row-major B) on two streams at once: each stream has its own
    repack scratch, so the results are those of the same calls made one after the other, bit for bit."""
    shapes = [(1536, 1280, 1024), (1280, 1536, 768)]
    g = torch.Generator(device="cuda").manual_seed(25)
    ops = []
    for (M, N, K) in shapes:
        A = torch.rand(M * K, device="cuda", generator=g) * 2 - 1
        B = torch.rand(K * N, device="cuda", generator=g) * 2 - 1
        alone = torch.empty(M * N, device="cuda")
        sgemm.gemm_3xtf32(0, 1, 0, alone, A, B, M, N, K)  # crr: both operands are repacked
        torch.cuda.synchronize()
        ops.append((M, N, K, A, B, alone, torch.full((M * N,), float("nan"), device="cuda")))
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    for _ in range(6):  # interleaved submissions, so that the two streams' kernels overlap on the GPU
        for s, (M, N, K, A, B, _, C) in zip(streams, ops):
            sgemm.gemm_3xtf32(0, 1, 0, C, A, B, M, N, K, stream=s)
    torch.cuda.synchronize()
    for (_, _, _, _, _, alone, C) in ops:
        assert torch.equal(C.view(torch.int32), alone.view(torch.int32))
    assert sgemm.tf32x3_device_status() == 0
