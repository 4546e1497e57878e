"""API breadth beside the drop-in entry: strided-batched products and the vendor-BLAS convention
(column-major C, transpose flags, leading dimensions, alpha / beta).  Both run the same kernels, so the bar stays
bit-exact against the CPU oracle's FMA chain (and, for alpha / beta, three separately rounded FP32 operations
restated with numpy float32 arithmetic)."""
import numpy as np
import pytest

from common import LAYOUTS, as2d, bits, layout_name

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def chain(sgemm, orc, lc, la, lb, A, B, M, N, K, batch=1):
    """The oracle's result with the split the table selects for this problem.  A batch never slices K (its matrices
    are the parallel work): every matrix of a batch is one k-ascending FMA chain per element."""
    if batch > 1:
        return orc.sgemm_fma(lc, la, lb, A, B, M, N, K, splits=1, threads=orc.max_threads())
    from common import oracle_chain
    sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return oracle_chain(sgemm, orc, la, lb, lc, A, B, M, N, K, sms)


@pytest.mark.parametrize("layout", [(0, 0, 0), (1, 0, 1), (0, 1, 0), (1, 1, 1)], ids=lambda l: layout_name(*l))
def test_strided_batched(sgemm, orc, layout):
    la, lb, lc = layout
    M, N, K, batch = 96, 130, 70, 3
    sa, sb, sc = M * K + 8, K * N, M * N + 4  # padded strides for A and C
    hostA = np.zeros(batch * sa, dtype=np.float32)
    hostB = np.zeros(batch * sb, dtype=np.float32)
    mats = []
    for b in range(batch):
        A, B = orc.fill_ab(30 + b, la, lb, M, N, K)
        hostA[b * sa:b * sa + M * K] = A
        hostB[b * sb:b * sb + K * N] = B
        mats.append((A, B))
    dA, dB = dev(hostA), dev(hostB)
    dC = torch.full((batch * sc,), float("nan"), device="cuda")
    sgemm.gemm_strided_batched(lc, la, lb, dC, dA, dB, M, N, K, sc, sa, sb, batch)
    torch.cuda.synchronize()
    C = dC.cpu().numpy()
    for b, (A, B) in enumerate(mats):
        want = chain(sgemm, orc, lc, la, lb, A, B, M, N, K, batch)
        assert np.array_equal(bits(C[b * sc:b * sc + M * N]), bits(want)), b
        assert np.isnan(C[b * sc + M * N:(b + 1) * sc]).all()  # the padding between matrices is untouched


def test_strided_batched_shared_operand_and_errors(sgemm, orc):
    M, N, K, batch = 64, 64, 32, 4
    A, B = orc.fill_ab(40, 0, 0, M, N, K)
    dA, dB = dev(A), dev(np.tile(B, batch))
    dC = torch.empty(batch * M * N, device="cuda")
    sgemm.gemm_strided_batched(0, 0, 0, dC, dA, dB, M, N, K, M * N, 0, K * N, batch)  # A shared (stride 0)
    torch.cuda.synchronize()
    want = chain(sgemm, orc, 0, 0, 0, A, B, M, N, K, batch)
    C = dC.cpu().numpy()
    for b in range(batch):
        assert np.array_equal(bits(C[b * M * N:(b + 1) * M * N]), bits(want))
    with pytest.raises(sgemm.SgemmError):
        sgemm.gemm_strided_batched(0, 0, 0, dC, dA, dB, M, N, K, M * N - 1, 0, K * N, batch)  # overlapping C
    with pytest.raises(sgemm.SgemmError):
        sgemm.gemm_strided_batched(0, 0, 0, dC, dA, dB, M, N, K, M * N, 0, K * N, 0)


@pytest.mark.parametrize("trans", [(0, 0), (1, 0), (0, 1), (1, 1)], ids=lambda t: "ta%d_tb%d" % t)
def test_blas_plain(sgemm, orc, trans):
    """alpha = 1, beta = 0: the reference's vendor-wrapper mapping, with padded leading dimensions."""
    ta, tb = trans
    M, N, K = 130, 70, 33
    la, lb = (0 if ta else 1), (0 if tb else 1)  # op(A) = A^T <=> the M x K operand is row-major
    A, B = orc.fill_ab(41, la, lb, M, N, K)
    lda = (K if ta else M) + 3
    ldb = (N if tb else K) + 5
    ldc = M + 2
    # embed the packed operands into padded storage (rows of the stored matrix have length ld)
    a_rows, a_len = (M, K) if ta else (K, M)
    b_rows, b_len = (K, N) if tb else (N, K)
    pA = np.full((a_rows, lda), np.nan, dtype=np.float32); pA[:, :a_len] = A.reshape(a_rows, a_len)
    pB = np.full((b_rows, ldb), np.nan, dtype=np.float32); pB[:, :b_len] = B.reshape(b_rows, b_len)
    dC = torch.full((N * ldc,), float("nan"), device="cuda")
    sgemm.gemm_blas(ta, tb, M, N, K, 1.0, dev(pA), lda, dev(pB), ldb, 0.0, dC, ldc)
    torch.cuda.synchronize()
    got = dC.cpu().numpy().reshape(N, ldc)
    want = chain(sgemm, orc, 1, la, lb, A, B, M, N, K).reshape(N, M)  # col-major C: N columns of M
    assert np.array_equal(bits(np.ascontiguousarray(got[:, :M])), bits(want))
    assert np.isnan(got[:, M:]).all()


@pytest.mark.parametrize("ab", [(2.5, 0.0), (1.0, 1.0), (-0.75, 0.5), (0.0, 2.0)], ids=lambda p: "a%g_b%g" % p)
def test_blas_alpha_beta(sgemm, orc, ab):
    alpha, beta = ab
    M, N, K = 257, 96, 64
    A, B = orc.fill_ab(42, 1, 1, M, N, K)  # col-major A and B: no transposes
    rng = np.random.default_rng(5)
    C0 = rng.uniform(-1, 1, M * N).astype(np.float32)
    dC = dev(C0.copy())
    sgemm.gemm_blas(0, 0, M, N, K, alpha, dev(A), M, dev(B), K, beta, dC, M)
    torch.cuda.synchronize()
    t = chain(sgemm, orc, 1, 1, 1, A, B, M, N, K)
    p = np.float32(alpha) * t                       # one FP32 rounding
    want = p if beta == 0.0 else p + np.float32(beta) * C0  # two more
    assert np.array_equal(bits(dC.cpu().numpy()), bits(want.astype(np.float32)))


def test_blas_beta_zero_ignores_nan_in_c(sgemm, orc):
    M, N, K = 64, 64, 32
    A, B = orc.fill_ab(43, 1, 1, M, N, K)
    dC = torch.full((M * N,), float("nan"), device="cuda")
    sgemm.gemm_blas(0, 0, M, N, K, 3.0, dev(A), M, dev(B), K, 0.0, dC, M)
    torch.cuda.synchronize()
    assert not torch.isnan(dC).any()


def test_blas_argument_errors(sgemm):
    x = torch.zeros(64, device="cuda")
    with pytest.raises(sgemm.SgemmError):
        sgemm.gemm_blas(0, 0, 8, 8, 8, 1.0, x, 7, x, 8, 0.0, x, 8)  # lda < M
    with pytest.raises(sgemm.SgemmError):
        sgemm.gemm_blas(1, 0, 8, 4, 8, 1.0, x, 8, x, 8, 0.0, x, 7)  # ldc < M
    with pytest.raises(sgemm.SgemmError):
        sgemm.gemm_blas(0, 0, 0, 8, 8, 1.0, x, 8, x, 8, 0.0, x, 8)


@pytest.mark.parametrize("lc", [0, 1], ids=["Crow", "Ccol"])
def test_multi_destination_store(sgemm, orc, lc):
    """b200_sgemm_multi: one kernel stores the result to several destinations (here three column blocks of full-size
    matrices on the same GPU, the single-GPU stand-in for the peers' copies of C)."""
    from rocm_sgemm_b200 import sharded
    M, N, K, world, rank = 192, 512, 96, 4, 2
    n = N // world
    la, lb = 1, 0
    A, B = orc.fill_ab(50, la, lb, M, n, K)
    full = [torch.full((M * N,), float("nan"), device="cuda") for _ in range(3)]
    off, ld = sharded.block_offset(lc, M, N, world, rank)
    dsts = [f.data_ptr() + 4 * off for f in full]
    sgemm.gemm_multi(lc, la, lb, dsts, dev(A), dev(B), M, n, K, ldc=ld)
    torch.cuda.synchronize()
    # this entry never splits K: one FMA chain per element
    want = as2d(orc.sgemm_fma(lc, la, lb, A, B, M, n, K, splits=1, threads=orc.max_threads()), lc, M, n)
    for f in full:
        got = as2d(f.cpu().numpy(), lc, M, N)
        assert np.array_equal(bits(np.ascontiguousarray(got[:, rank * n:(rank + 1) * n])), bits(np.ascontiguousarray(want)))
        rest = np.delete(got, np.s_[rank * n:(rank + 1) * n], axis=1)
        assert np.isnan(rest).all()  # nothing outside the block is touched
    with pytest.raises(sgemm.SgemmError):
        sgemm.gemm_multi(lc, la, lb, [], dev(A), dev(B), M, n, K, ldc=ld)
    with pytest.raises(sgemm.SgemmError):
        sgemm.gemm_multi(lc, la, lb, [dsts[0]] * 9, dev(A), dev(B), M, n, K, ldc=ld)


@pytest.mark.parametrize("layout", [(0, 0, 0), (1, 0, 0), (0, 1, 1), (1, 1, 0)], ids=lambda l: layout_name(*l))
@pytest.mark.parametrize("case", [(512, 384, 256, 8, 0), (320, 512, 130, 5, 0), (256, 256, 512, 37, 0), (200, 136, 132, 6, 3)],
                         ids=lambda c: "x".join(map(str, c)))
def test_strided_batched_one_launch(sgemm, orc, case, layout):
    """Batches large enough to be worth one launch: the persistent CTAs walk the tiles of all matrices (with the
    hand-over schedule when batch x tiles exceeds the SMs).  Every matrix must be the oracle's single FMA chain, bit
    for bit; `pad` > 0 makes the strides odd, which sends the operands through the kernel's guarded route."""
    (M, N, K, batch, pad), (la, lb, lc) = case, layout
    sa, sb, sc = M * K + pad, K * N + pad, M * N + pad
    hostA = np.zeros(batch * sa, dtype=np.float32)
    hostB = np.zeros(batch * sb, dtype=np.float32)
    A0, B0 = orc.fill_ab(50, la, lb, M, N, K)
    rng = np.random.default_rng(51)
    mats = []
    for b in range(batch):
        A = (A0 * np.float32(1 + 0.125 * b)).astype(np.float32) if b % 2 else rng.uniform(-1, 1, M * K).astype(np.float32)
        B = B0 if b % 3 else rng.uniform(-1, 1, K * N).astype(np.float32)
        hostA[b * sa:b * sa + M * K] = A
        hostB[b * sb:b * sb + K * N] = B
        mats.append((A, B))
    dA, dB = dev(hostA), dev(hostB)
    dC = torch.full((batch * sc,), float("nan"), device="cuda")
    sgemm.gemm_strided_batched(lc, la, lb, dC, dA, dB, M, N, K, sc, sa, sb, batch)
    torch.cuda.synchronize()
    C = dC.cpu().numpy()
    for b in (0, 1, batch // 2, batch - 1):
        A, B = mats[b]
        want = chain(sgemm, orc, lc, la, lb, A, B, M, N, K, batch)
        assert np.array_equal(bits(C[b * sc:b * sc + M * N]), bits(want)), b
    if pad:
        for b in range(batch):
            assert np.isnan(C[b * sc + M * N:(b + 1) * sc]).all()
    assert sgemm.device_status() == 0
