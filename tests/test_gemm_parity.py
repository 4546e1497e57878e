"""GPU parity of the CUDA SGEMM path, called through the C ABI, against the CPU oracle.

Bars (stated per test):
  * bit-exact against the oracle's k-ascending FMA chain (oracle.sgemm_fma), the arithmetic the
    kernels are specified to perform, including the ordered split-K sum;
  * |c - c_ref| <= 1e-4 absolute against the reference's sgemm_cpu restatement, the tolerance of the
    reference's own suite (test/gemm/test.cpp:82-90);
  * max relative error against a float64 accumulation <= 1e-5 * sqrt(K), and no worse than the
    reference's CPU GEMM on the same inputs (rms error <= 1.02x, max error <= 2x: the maxima of two
    different rounding sequences are random variables, the rms is the stable comparison);
  * bit-exact C == A for the identity-B configuration.
"""
import math

import numpy as np
import pytest

from common import LAYOUTS, REFERENCE_TEST_SHAPES, SWEEP_SHAPES, as2d, bits, layout_name, oracle_chain

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def dev(a: np.ndarray):
    return torch.from_numpy(a).cuda()


def run_gemm(sgemm, la, lb, lc, A, B, M, N, K, **ex):
    """A, B packed host arrays -> packed host C through b200_sgemm (or b200_sgemm_ex when `ex` given)."""
    dA, dB = dev(A), dev(B)
    dC = torch.full((M * N,), float("nan"), dtype=torch.float32, device="cuda")
    if ex:
        ws = None
        nbytes = sgemm.workspace_bytes(lc, la, lb, M, N, K, ex.get("variant", -1), ex.get("split_k", 0))
        if nbytes:
            ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        sgemm.gemm_ex(lc, la, lb, dC, dA, dB, M, N, K, workspace=ws, workspace_bytes=nbytes, **ex)
    else:
        sgemm.gemm(lc, la, lb, dC, dA, dB, M, N, K)
    torch.cuda.synchronize()
    return dC.cpu().numpy()


def effective_split(sgemm, la, lb, lc, M, N, K, variant=-1, split_k=0):
    """(splits, block_k) the library will use, for the oracle's split-K restatement."""
    p, v = sgemm.select_config(M, N, K, lc, la, lb)
    if variant >= 0:
        p = sgemm.get_variant(variant)
    s = split_k if split_k > 0 else (p.split_k if variant < 0 else 1)
    return s, p.block_k


def sm_count():
    return torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count


def expect_bit_exact(sgemm, orc, la, lb, lc, A, B, M, N, K, C, rows=None, **ex):
    want = oracle_chain(sgemm, orc, la, lb, lc, A, B, M, N, K, sm_count(), rows, ex.get("variant", -1),
                        ex.get("split_k", 0))
    got, want2 = as2d(C, lc, M, N), as2d(want, lc, M, N)
    if rows is not None:
        got, want2 = got[rows[0]:rows[1]], want2[rows[0]:rows[1]]
    bad = np.argwhere(bits(np.ascontiguousarray(got)) != bits(np.ascontiguousarray(want2)))
    assert bad.size == 0, f"{len(bad)} elements differ from the FMA-chain oracle, first at {bad[0]}: " \
                          f"{got[tuple(bad[0])]} vs {want2[tuple(bad[0])]}"


# ------------------------------------------------------------------------------------------------
# the reference's own suite: 13 shapes x 8 layouts, mt19937(1) inputs re-seeded per matrix
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("layout", LAYOUTS, ids=lambda l: layout_name(*l))
@pytest.mark.parametrize("shape", REFERENCE_TEST_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_reference_suite(sgemm, orc, shape, layout):
    (M, N, K), (la, lb, lc) = shape, layout
    A, B = orc.init_matrix(la, M, K), orc.init_matrix(lb, K, N)
    C = run_gemm(sgemm, la, lb, lc, A, B, M, N, K)
    ref = orc.sgemm_f32(lc, la, lb, A, B, M, N, K, threads=orc.max_threads())
    assert np.max(np.abs(C - ref)) <= 1e-4  # the reference suite's tolerance
    expect_bit_exact(sgemm, orc, la, lb, lc, A, B, M, N, K, C)


# ------------------------------------------------------------------------------------------------
# benchmark configuration 1: 256^3 row-major, seed 0, against float64
# ------------------------------------------------------------------------------------------------
def check_against_f64(orc, la, lb, lc, A, B, M, N, K, C, rows=None):
    ref64 = orc.sgemm_f64(lc, la, lb, A, B, M, N, K, rows=rows, threads=orc.max_threads())
    cpu = orc.sgemm_f32(lc, la, lb, A, B, M, N, K, rows=rows, threads=orc.max_threads())
    e_gpu = orc.error_metrics(lc, C, ref64, M, N, rows=rows)
    e_cpu = orc.error_metrics(lc, cpu, ref64, M, N, rows=rows)
    tol = 1e-5 * math.sqrt(K)
    assert e_gpu["max_rel"] <= tol, (e_gpu, tol)
    assert e_gpu["rms_err"] <= 1.02 * e_cpu["rms_err"] + 1e-12, (e_gpu, e_cpu)
    assert e_gpu["max_rel"] <= 2.0 * e_cpu["max_rel"] + 1e-12, (e_gpu, e_cpu)
    return e_gpu, e_cpu


def test_config1_256_cube(sgemm, orc):
    M = N = K = 256
    A, B = orc.fill_ab(0, 0, 0, M, N, K)
    C = run_gemm(sgemm, 0, 0, 0, A, B, M, N, K)
    check_against_f64(orc, 0, 0, 0, A, B, M, N, K, C)
    expect_bit_exact(sgemm, orc, 0, 0, 0, A, B, M, N, K, C)


# ------------------------------------------------------------------------------------------------
# benchmark configuration 2: identity B, C must equal A bit for bit (all layouts, full size)
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("layout", LAYOUTS, ids=lambda l: layout_name(*l))
def test_config2_identity_bit_exact(sgemm, orc, layout):
    la, lb, lc = layout
    M = N = K = 4096
    A, _ = orc.fill_ab(1, la, lb, M, N, K, with_b=False)
    I = orc.fill_identity(lb, K, N)
    C = run_gemm(sgemm, la, lb, lc, A, I, M, N, K)
    assert np.array_equal(bits(np.ascontiguousarray(as2d(C, lc, M, N))), bits(np.ascontiguousarray(as2d(A, la, M, K))))


# ------------------------------------------------------------------------------------------------
# benchmark configuration 3: 4096^3 in all eight layouts, seed 2
# ------------------------------------------------------------------------------------------------
def full_check_f64_on_device(la, lb, lc, A, B, M, N, K, C, tol):
    """Whole-matrix check at full size against a float64 product evaluated on the device."""
    A2 = dev(A).view(M, K) if la == 0 else dev(A).view(K, M).T
    B2 = dev(B).view(K, N) if lb == 0 else dev(B).view(N, K).T
    ref = A2.double() @ B2.double()
    C2 = dev(C).view(M, N) if lc == 0 else dev(C).view(N, M).T
    rms = ref.pow(2).mean().sqrt()
    rel = ((C2.double() - ref).abs() / torch.maximum(ref.abs(), rms)).max().item()
    assert rel <= tol, rel
    return rel


@pytest.mark.parametrize("layout", LAYOUTS, ids=lambda l: layout_name(*l))
def test_config3_4096_all_layouts(sgemm, orc, layout):
    la, lb, lc = layout
    M = N = K = 4096
    A, B = orc.fill_ab(2, la, lb, M, N, K)
    C = run_gemm(sgemm, la, lb, lc, A, B, M, N, K)
    rows = (1000, 1016)  # a band of full rows through the oracle, the whole matrix on the device
    check_against_f64(orc, la, lb, lc, A, B, M, N, K, C, rows=rows)
    expect_bit_exact(sgemm, orc, la, lb, lc, A, B, M, N, K, C, rows=rows)
    full_check_f64_on_device(la, lb, lc, A, B, M, N, K, C, 1e-5 * math.sqrt(K))


# ------------------------------------------------------------------------------------------------
# benchmark configuration 4: rectangular / skinny sweep, row-major, seed 3 (table + split-K)
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("shape", SWEEP_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_config4_sweep(sgemm, orc, shape):
    M, N, K = shape
    A, B = orc.fill_ab(3, 0, 0, M, N, K)
    C = run_gemm(sgemm, 0, 0, 0, A, B, M, N, K)
    r0 = M // 3
    rows = (r0, r0 + 8)
    check_against_f64(orc, 0, 0, 0, A, B, M, N, K, C, rows=rows)
    expect_bit_exact(sgemm, orc, 0, 0, 0, A, B, M, N, K, C, rows=rows)
    full_check_f64_on_device(0, 0, 0, A, B, M, N, K, C, 1e-5 * math.sqrt(K))


# ------------------------------------------------------------------------------------------------
# benchmark configuration 5 on one GPU: 16384^3, N(0,1) from seed 4 generated on the device
# ------------------------------------------------------------------------------------------------
def test_config5_16384_single_gpu(sgemm, orc):
    M = N = K = 16384
    g = torch.Generator(device="cuda")
    g.manual_seed(4)
    dA = torch.randn(M * K, generator=g, dtype=torch.float32, device="cuda")
    dB = torch.randn(K * N, generator=g, dtype=torch.float32, device="cuda")
    dC = torch.empty(M * N, dtype=torch.float32, device="cuda")
    sgemm.gemm(0, 0, 0, dC, dA, dB, M, N, K)
    torch.cuda.synchronize()
    tol = 1e-5 * math.sqrt(K)
    # bands of rows against a float64 product on the device
    for r0 in (0, 5000, 16384 - 64):
        ref = dA.view(M, K)[r0:r0 + 64].double() @ dB.view(K, N).double()
        got = dC.view(M, N)[r0:r0 + 64].double()
        rms = ref.pow(2).mean().sqrt()
        assert ((got - ref).abs() / torch.maximum(ref.abs(), rms)).max().item() <= tol
    # four rows through the oracle's FMA chain, bit for bit
    A, B = dA.cpu().numpy(), dB.cpu().numpy()
    C = dC.cpu().numpy()
    expect_bit_exact(sgemm, orc, 0, 0, 0, A, B, M, N, K, C, rows=(7777, 7781))


# ------------------------------------------------------------------------------------------------
# ragged and degenerate shapes (the reference's loads are unguarded there; this library is exact)
# ------------------------------------------------------------------------------------------------
# the last three are large enough in M or N for the drop-in entry to pre-transpose a K-contiguous operand
RAGGED = [(1, 1, 1), (3, 5, 7), (1, 300, 40), (300, 1, 40), (127, 129, 65), (130, 70, 33), (257, 255, 100),
          (33, 1000, 17), (64, 64, 1), (200, 136, 132), (130, 1101, 70), (1101, 130, 70), (1027, 1030, 37)]


@pytest.mark.parametrize("layout", LAYOUTS, ids=lambda l: layout_name(*l))
@pytest.mark.parametrize("shape", RAGGED, ids=lambda s: "x".join(map(str, s)))
def test_ragged_shapes(sgemm, orc, shape, layout):
    (M, N, K), (la, lb, lc) = shape, layout
    A, B = orc.fill_ab(5, la, lb, M, N, K)
    C = run_gemm(sgemm, la, lb, lc, A, B, M, N, K)
    expect_bit_exact(sgemm, orc, la, lb, lc, A, B, M, N, K, C)


def test_guard_bands_untouched(sgemm, orc):
    """C is written only inside its M x N extent: sentinel bands before and after stay intact."""
    for (la, lb, lc) in [(0, 0, 0), (1, 1, 1), (0, 1, 0), (1, 0, 1)]:
        M, N, K = 130, 75, 50
        A, B = orc.fill_ab(6, la, lb, M, N, K)
        pad = 512
        buf = torch.full((M * N + 2 * pad,), -12345.0, dtype=torch.float32, device="cuda")
        sgemm.gemm(lc, la, lb, buf[pad:], dev(A), dev(B), M, N, K)
        torch.cuda.synchronize()
        h = buf.cpu().numpy()
        assert (h[:pad] == -12345.0).all() and (h[-pad:] == -12345.0).all()
        expect_bit_exact(sgemm, orc, la, lb, lc, A, B, M, N, K, h[pad:-pad].copy())


# ------------------------------------------------------------------------------------------------
# split-K: ordered, deterministic, bit-exact against the oracle's split restatement
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("layout", [(0, 0, 0), (1, 1, 1), (0, 1, 0), (1, 0, 1)], ids=lambda l: layout_name(*l))
@pytest.mark.parametrize("split", [2, 3, 7, 16])
def test_split_k(sgemm, orc, layout, split):
    la, lb, lc = layout
    for (M, N, K) in [(64, 64, 4096), (130, 70, 1000)]:
        A, B = orc.fill_ab(8, la, lb, M, N, K)
        C1 = run_gemm(sgemm, la, lb, lc, A, B, M, N, K, split_k=split)
        C2 = run_gemm(sgemm, la, lb, lc, A, B, M, N, K, split_k=split)
        assert np.array_equal(bits(C1), bits(C2))  # no atomics: run-to-run identical
        expect_bit_exact(sgemm, orc, la, lb, lc, A, B, M, N, K, C1, split_k=split)


def test_split_k_through_drop_in_entry(sgemm, orc):
    """A tabled skinny problem takes the split-K route inside b200_sgemm (internal arena)."""
    entries = [e for e in sgemm.table_entries() if e[7] > 1]
    if not entries:
        pytest.skip("the shipped table has no split-K entry")
    M, N, K, la, lb, lc, _, s = entries[0]
    A, B = orc.fill_ab(9, la, lb, M, N, K)
    C = run_gemm(sgemm, la, lb, lc, A, B, M, N, K)
    r0 = M // 2
    expect_bit_exact(sgemm, orc, la, lb, lc, A, B, M, N, K, C, rows=(r0, r0 + 4))


# ------------------------------------------------------------------------------------------------
# leading dimensions (the entry the column-sharded driver uses)
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("layout", LAYOUTS, ids=lambda l: layout_name(*l))
def test_leading_dimensions(sgemm, orc, layout):
    la, lb, lc = layout
    M, N, K = 192, 160, 96
    A, B = orc.fill_ab(10, la, lb, M, N, K)
    lda = (K if la == 0 else M) + 12
    ldb = (N if lb == 0 else K) + 8
    ldc = (N if lc == 0 else M) + 20

    def embed(flat, layout, rows, cols, ld):
        outer, inner = (rows, cols) if layout == 0 else (cols, rows)
        buf = np.full((outer, ld), 777.0, dtype=np.float32)
        buf[:, :inner] = flat.reshape(outer, inner)
        return buf

    dA, dB = dev(embed(A, la, M, K, lda)), dev(embed(B, lb, K, N, ldb))
    outer_c, inner_c = (M, N) if lc == 0 else (N, M)
    dC = torch.full((outer_c, ldc), -1.0, dtype=torch.float32, device="cuda")
    for split in (1, 3):
        nbytes = sgemm.workspace_bytes(lc, la, lb, M, N, K, -1, split)
        ws = torch.empty(max(nbytes, 1), dtype=torch.uint8, device="cuda")
        dC.fill_(-1.0)
        sgemm.gemm_ex(lc, la, lb, dC, dA, dB, M, N, K, lda=lda, ldb=ldb, ldc=ldc, split_k=split, workspace=ws,
                      workspace_bytes=nbytes)
        torch.cuda.synchronize()
        h = dC.cpu().numpy()
        assert (h[:, inner_c:] == -1.0).all()  # the padding columns of C are not written
        expect_bit_exact(sgemm, orc, la, lb, lc, A, B, M, N, K, np.ascontiguousarray(h[:, :inner_c]).ravel(),
                         split_k=split)


# ------------------------------------------------------------------------------------------------
# every kernel built into the library (tuned variants x layouts x aligned/unaligned)
# ------------------------------------------------------------------------------------------------
def test_every_built_kernel(sgemm, orc):
    checked = 0
    for v in range(sgemm.num_variants()):
        p = sgemm.get_variant(v)
        for (la, lb, lc) in LAYOUTS:
            if not sgemm.has_kernel(v, la, lb, lc, True):
                continue
            for (M, N, K) in [(2 * p.block_m, 2 * p.block_n, 4 * p.block_k),  # aligned kernel
                              (p.block_m + 5, 2 * p.block_n - 3, 3 * p.block_k + 2)]:  # unaligned kernel
                A, B = orc.fill_ab(12, la, lb, M, N, K)
                C = run_gemm(sgemm, la, lb, lc, A, B, M, N, K, variant=v, split_k=1)
                expect_bit_exact(sgemm, orc, la, lb, lc, A, B, M, N, K, C, variant=v, split_k=1)
                checked += 1
    assert checked >= 16


def test_unaligned_pointers(sgemm, orc):
    """Device pointers that are only 4-byte aligned take the scalar path and stay exact."""
    M, N, K = 96, 80, 64
    for (la, lb, lc) in [(0, 0, 0), (1, 1, 1), (1, 0, 0), (0, 1, 1)]:
        A, B = orc.fill_ab(13, la, lb, M, N, K)
        bufA = torch.zeros(M * K + 1, dtype=torch.float32, device="cuda")
        bufB = torch.zeros(K * N + 1, dtype=torch.float32, device="cuda")
        bufC = torch.zeros(M * N + 1, dtype=torch.float32, device="cuda")
        bufA[1:] = dev(A)
        bufB[1:] = dev(B)
        sgemm.gemm(lc, la, lb, bufC[1:], bufA[1:], bufB[1:], M, N, K)
        torch.cuda.synchronize()
        expect_bit_exact(sgemm, orc, la, lb, lc, A, B, M, N, K, bufC[1:].cpu().numpy())


def test_stream_argument(sgemm, orc):
    M, N, K = 128, 128, 64
    A, B = orc.fill_ab(14, 0, 0, M, N, K)
    dA, dB = dev(A), dev(B)
    dC = torch.zeros(M * N, dtype=torch.float32, device="cuda")
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    sgemm.gemm(0, 0, 0, dC, dA, dB, M, N, K, stream=s)
    s.synchronize()
    expect_bit_exact(sgemm, orc, 0, 0, 0, A, B, M, N, K, dC.cpu().numpy())


def test_fma_probe_runs(sgemm):
    for mode in (0, 1):
        r = sgemm.fma_peak(mode, 512)
        assert r["ms"] > 0 and 1.0 < r["tflops"] < 200.0


def test_device_status_clean(sgemm):
    """No kernel launched by this module gave up a bounded wait."""
    assert sgemm.device_status() == 0


# ------------------------------------------------------------------------------------------------
# host-buffer entry: upload, GEMM and download pipelined in one call
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("layout", LAYOUTS, ids=lambda l: layout_name(*l))
def test_host_buffer_entry(sgemm, orc, layout):
    la, lb, lc = layout
    for (M, N, K) in [(2304, 320, 96), (130, 70, 33), (1024, 128, 64)]:  # several panels / one ragged panel
        A, B = orc.fill_ab(15, la, lb, M, N, K)
        hA, hB = torch.from_numpy(A).pin_memory(), torch.from_numpy(B).pin_memory()
        hC = torch.full((M * N,), float("nan"), dtype=torch.float32).pin_memory()
        sgemm.gemm_host(lc, la, lb, hC, hA, hB, M, N, K)
        p, _ = sgemm.select_config(M, N, K, lc, la, lb)
        want = orc.sgemm_fma(lc, la, lb, A, B, M, N, K, splits=1, k_align=p.block_k, threads=orc.max_threads())
        assert np.array_equal(bits(hC.numpy()), bits(want)), (layout, (M, N, K))
    # pageable host memory works too (without the overlap)
    M, N, K = 300, 200, 64
    A, B = orc.fill_ab(16, la, lb, M, N, K)
    C = np.empty(M * N, dtype=np.float32)
    sgemm.gemm_host(lc, la, lb, C.ctypes.data, A.ctypes.data, B.ctypes.data, M, N, K)
    assert np.array_equal(bits(C), bits(orc.sgemm_fma(lc, la, lb, A, B, M, N, K)))


@pytest.mark.parametrize("layout", LAYOUTS, ids=lambda l: layout_name(*l))
def test_host_buffer_entry_strips(sgemm, orc, layout):
    """Large problems are computed as rectangular strips (A row panels x B column panels, split-K per
    strip).  Identity B gives C == A bit for bit under any split; random inputs meet the float64 bound."""
    la, lb, lc = layout
    M, N, K = 2304, 1280, 1280  # 4 x 2 pieces of 640, the last row panel shorter
    A, _ = orc.fill_ab(17, la, lb, M, N, K, with_b=False)
    I = orc.fill_identity(lb, K, N)
    hA, hI = torch.from_numpy(A).pin_memory(), torch.from_numpy(I).pin_memory()
    hC = torch.full((M * N,), float("nan"), dtype=torch.float32).pin_memory()
    sgemm.gemm_host(lc, la, lb, hC, hA, hI, M, N, K)
    assert np.array_equal(bits(np.ascontiguousarray(as2d(hC.numpy(), lc, M, N))),
                          bits(np.ascontiguousarray(as2d(A, la, M, K))))
    M, N, K = 1100, 1536, 1024  # ragged M
    A, B = orc.fill_ab(18, la, lb, M, N, K)
    hA, hB = torch.from_numpy(A).pin_memory(), torch.from_numpy(B).pin_memory()
    hC = torch.full((M * N,), float("nan"), dtype=torch.float32).pin_memory()
    sgemm.gemm_host(lc, la, lb, hC, hA, hB, M, N, K)
    full_check_f64_on_device(la, lb, lc, A, B, M, N, K, hC.numpy(), 1e-5 * math.sqrt(K))
    # every strip is an ordered split-K sum of FMA chains: the plain chain is within a few ulp of it
    want = orc.sgemm_fma(lc, la, lb, A, B, M, N, K, threads=orc.max_threads())
    assert np.max(np.abs(hC.numpy() - want)) <= 1e-4


def test_host_buffer_submit_wait(sgemm, orc):
    """Asynchronous form of the host-buffer entry: several jobs submitted back to back (two in flight, the third
    submit waits for the first), tickets awaited in and out of order, every result bit-exact."""
    la, lb, lc = 0, 0, 0
    shapes = [(1100, 1536, 1024), (300, 200, 64), (2304, 1280, 1280), (130, 70, 33), (1024, 1024, 1024)]
    jobs = []
    for i, (M, N, K) in enumerate(shapes):
        A, B = orc.fill_ab(70 + i, la, lb, M, N, K)
        hA, hB = torch.from_numpy(A).pin_memory(), torch.from_numpy(B).pin_memory()
        hC = torch.full((M * N,), float("nan"), dtype=torch.float32).pin_memory()
        t = sgemm.gemm_host_submit(lc, la, lb, hC, hA, hB, M, N, K)
        jobs.append((t, (M, N, K), A, B, hA, hB, hC))
    assert [j[0] for j in jobs] == list(range(jobs[0][0], jobs[0][0] + len(jobs)))
    for j in (jobs[3], jobs[4], jobs[0], jobs[2], jobs[1]):  # any order; finished tickets return at once
        sgemm.gemm_host_wait(j[0])
    sgemm.gemm_host_wait(jobs[0][0])  # waiting twice is harmless
    for t, (M, N, K), A, B, hA, hB, hC in jobs:
        full_check_f64_on_device(la, lb, lc, A, B, M, N, K, hC.numpy(), 1e-5 * math.sqrt(K))
        if M < 1024:  # small problems run unsplit: bit-exact against the plain chain
            want = orc.sgemm_fma(lc, la, lb, A, B, M, N, K, threads=orc.max_threads())
            assert np.array_equal(bits(hC.numpy()), bits(want))
    with pytest.raises(sgemm.SgemmError):
        sgemm.gemm_host_wait(jobs[-1][0] + 1000)  # never issued


def test_reentrant_threads_and_streams(sgemm, orc):
    """Four host threads, each with its own stream, call the drop-in entry concurrently (split-K and pre-transposing
    table entries included, so the per-(device, stream) arenas are in play); every result stays bit-exact."""
    import threading
    cases = [((1024, 1024, 1024), (0, 1, 0)), ((1027, 1030, 37), (1, 0, 1)), ((2048, 2048, 2048), (0, 0, 0)),
             ((300, 200, 4096), (1, 1, 0))]
    inputs = []
    for i, ((M, N, K), (la, lb, lc)) in enumerate(cases):
        A, B = orc.fill_ab(80 + i, la, lb, M, N, K)
        inputs.append((dev(A), dev(B), torch.full((M * N,), float("nan"), device="cuda"), A, B))
    errors = []

    def work(i):
        try:
            (M, N, K), (la, lb, lc) = cases[i]
            dA, dB, dC, _, _ = inputs[i]
            s = torch.cuda.Stream()
            for _ in range(6):
                sgemm.gemm(lc, la, lb, dC, dA, dB, M, N, K, stream=s)
            s.synchronize()
        except Exception as ex:  # surfaced in the main thread below
            errors.append((i, repr(ex)))

    threads = [threading.Thread(target=work, args=(i,)) for i in range(len(cases))]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    torch.cuda.synchronize()
    for i, ((M, N, K), (la, lb, lc)) in enumerate(cases):
        _, _, dC, A, B = inputs[i]
        expect_bit_exact(sgemm, orc, la, lb, lc, A, B, M, N, K, dC.cpu().numpy())
    assert sgemm.device_status() == 0


def test_bounded_wait_gives_up_and_reports(sgemm):
    """The time-out path of the kernels' waits, made to happen without any fault: the self-test launches a private copy
    of the warp-specialised kernel (wait limit 1 ms) on one tile and withholds the last K tile, so the consumer
    warps' wait for that stage runs out.  Every thread returns, the status word reads 1 (consumer-side time-out) once
    and 0 afterwards, C is untouched, and the device computes correctly right after."""
    dA = torch.rand(128 * 64, dtype=torch.float32, device="cuda")
    dB = torch.rand(64 * 128, dtype=torch.float32, device="cuda")
    dC = torch.full((128 * 128,), 7.0, dtype=torch.float32, device="cuda")
    assert sgemm.device_status() == 0
    sgemm.selftest_bounded_wait(dC, dA, dB)
    torch.cuda.synchronize()  # the kernel ended by itself
    assert sgemm.device_status() == 1
    assert sgemm.device_status() == 0
    assert bool((dC == 7.0).all())
    # the context is healthy: an ordinary product right after is exact
    sgemm.gemm(0, 1, 0, dC, dA, dB, 128, 128, 64)
    torch.cuda.synchronize()
    ref = dA.view(64, 128).T.double() @ dB.view(64, 128).double()
    assert float((dC.view(128, 128).double() - ref).abs().max()) < 1e-4
    assert sgemm.device_status() == 0


@pytest.mark.parametrize("layout", [(0, 0, 0), (0, 1, 0), (1, 1, 1), (0, 1, 1)], ids=lambda l: layout_name(*l))
@pytest.mark.parametrize("shape", [(1024, 1024, 512), (1028, 1100, 1036), (1152, 1026, 260)],
                         ids=lambda s: "x".join(map(str, s)))
def test_transposition_inside_the_kernel(sgemm, orc, shape, layout):
    """Entries with pretranspose bits multiply a K-contiguous operand from a transposed copy.  The warp-specialised
    kernels make that copy themselves (idle producer warps transpose it block by block, the copy-issuing thread
    waits for the blocks a stage needs); bit 2 of a trial's pretranspose argument asks for the transposition kernel
    in front of the product instead.  Both must give the oracle's single FMA chain bit for bit.  The second shape
    has ragged tiles in every dimension; in the third N is not a multiple of 4, so a column-major B cannot be
    transposed inside and the library falls back to the kernel in front by itself."""
    (M, N, K), (la, lb, lc) = shape, layout
    pre = (1 if la == 0 else 0) | (2 if lb == 1 else 0)
    variant = None
    for i in range(sgemm.num_variants()):
        p = sgemm.get_variant(i)
        if ((p.pipeline, p.block_m, p.block_n, p.block_k, p.block_size) == (1, 128, 128, 32, 256)
                and all(sgemm.has_kernel(i, a, b, lc, al) for a, b in ((la, lb), (1, lb), (1, 0), (la, 0)) for al in (True, False))):
            variant = i
            break
    if variant is None:
        pytest.skip("no 128x128x32 warp-specialised variant built for this layout and its transposed forms")
    A, B = orc.fill_ab(61, la, lb, M, N, K)
    dA, dB = dev(A), dev(B)
    got = []
    for bits_ in (pre, pre | 4):
        dC = torch.full((M * N,), float("nan"), dtype=torch.float32, device="cuda")
        for _ in range(2):  # twice: the second call finds the flag words of the first (an older epoch)
            sgemm.gemm_trial(lc, la, lb, dC, dA, dB, M, N, K, variant, 1, bits_)
        torch.cuda.synchronize()
        got.append(dC.cpu().numpy())
    want = orc.sgemm_fma(lc, la, lb, A, B, M, N, K, splits=1, threads=orc.max_threads())
    assert np.array_equal(bits(got[0]), bits(want))
    assert np.array_equal(bits(got[1]), bits(want))
    assert sgemm.device_status() == 0


def test_release_stream_frees_the_arena(sgemm, orc):
    """b200_sgemm_release_stream: the scratch the drop-in entry keeps for a stream goes back to the device (seen in
    cudaMemGetInfo), a stream the library has never seen is not an error, and the next call on the stream simply
    allocates again and gives the same bits."""
    M, N, K = 1024, 1024, 16384  # the tabled skinny problem: parking slots in the arena
    A, B = orc.fill_ab(71, 0, 0, M, N, K)
    dA, dB = dev(A), dev(B)
    dC = torch.empty(M * N, dtype=torch.float32, device="cuda")
    s = torch.cuda.Stream()
    sgemm.release_stream(s)  # unknown stream
    with torch.cuda.stream(s):
        sgemm.gemm(0, 0, 0, dC, dA, dB, M, N, K, stream=s)
    s.synchronize()
    first = dC.clone()
    held, _ = torch.cuda.mem_get_info()
    sgemm.release_stream(s)
    freed, _ = torch.cuda.mem_get_info()
    assert freed - held >= 1024 * 1024  # at least the arena's flag words came back
    dC.fill_(float("nan"))
    with torch.cuda.stream(s):
        sgemm.gemm(0, 0, 0, dC, dA, dB, M, N, K, stream=s)
    s.synchronize()
    assert torch.equal(dC.view(torch.int32), first.view(torch.int32))
    sgemm.release_stream(s)
    assert sgemm.device_status() == 0


def test_transposition_inside_the_kernel_is_repeatable(sgemm, orc):
    """The flag-word hand-over between the transposing warps and the thread that issues the TMA copies, exercised many
    times: 40 calls on a problem with 2 x 16 x 64 blocks must all give the bits of the transposition kernel in front
    (a block read before it was complete would show as a difference)."""
    M = N = K = 2048
    la, lb, lc = 0, 1, 0
    variant = None
    for i in range(sgemm.num_variants()):
        p = sgemm.get_variant(i)
        if ((p.pipeline, p.block_m, p.block_n, p.block_k, p.block_size) == (1, 128, 128, 32, 256)
                and all(sgemm.has_kernel(i, a, b, lc, True) for a, b in ((0, 1), (1, 1), (1, 0), (0, 0)))):
            variant = i
            break
    if variant is None:
        pytest.skip("no 128x128x32 warp-specialised variant built for rcr and its transposed forms")
    g = torch.Generator(device="cuda").manual_seed(81)
    dA = torch.rand(M * K, generator=g, device="cuda") * 2 - 1
    dB = torch.rand(K * N, generator=g, device="cuda") * 2 - 1
    ref = torch.empty(M * N, device="cuda")
    sgemm.gemm_trial(lc, la, lb, ref, dA, dB, M, N, K, variant, 1, 3 | 4)
    out = [torch.full((M * N,), float("nan"), device="cuda") for _ in range(4)]
    for rep in range(40):
        sgemm.gemm_trial(lc, la, lb, out[rep % 4], dA, dB, M, N, K, variant, 1, 3)
        if rep % 4 == 3:
            for o in out:
                assert torch.equal(o.view(torch.int32), ref.view(torch.int32)), rep
                o.fill_(float("nan"))
    assert sgemm.device_status() == 0
