"""The balanced schedules of the warp-specialised kernel against the oracle, through the C ABI.

* Schedule with one accumulator hand-over (at least as many tiles as SMs): every C element stays ONE k-ascending
  FMA chain, so the result must equal the unsplit oracle chain bit for bit, and equal the round-robin schedule's.
* Equal K ranges with in-kernel ordered reduction (fewer tiles than SMs; split_k -1 / table entries with split_k 0):
  the result must equal, bit for bit, the oracle's ordered sum of chains over the K cut points the library reports
  (b200_sgemm_stream_plan), and meet the float64 bound 1e-5 * sqrt(K).
"""
import math

import numpy as np
import pytest

from common import as2d, bits, layout_name, oracle_chain

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

WS_VARIANTS = {}


def ws_variant(sgemm, la=0, lb=0, lc=0):
    """A 128 x 128 x 32 warp-specialised variant of the shipped table that is built for this layout (variants are
    compiled only for the layouts whose table entries name them)."""
    key = (la, lb, lc)
    if key not in WS_VARIANTS:
        for i in range(sgemm.num_variants()):
            p = sgemm.get_variant(i)
            if ((p.pipeline, p.block_m, p.block_n, p.block_k, p.block_size) == (1, 128, 128, 32, 256)
                    and sgemm.has_kernel(i, la, lb, lc, True) and sgemm.has_kernel(i, la, lb, lc, False)):
                WS_VARIANTS[key] = i
                break
    assert key in WS_VARIANTS, "no 128x128x32 warp-specialised kernel for layout %s" % (key,)
    return WS_VARIANTS[key]


def sms():
    return torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count


def run_ex(sgemm, la, lb, lc, A, B, M, N, K, variant, split_k, with_workspace=True):
    dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    dC = torch.full((M * N,), float("nan"), dtype=torch.float32, device="cuda")
    nbytes = sgemm.workspace_bytes(lc, la, lb, M, N, K, variant, split_k) if with_workspace else 0
    ws = torch.empty(max(nbytes, 1), dtype=torch.uint8, device="cuda") if nbytes else None
    sgemm.gemm_ex(lc, la, lb, dC, dA, dB, M, N, K, variant=variant, split_k=split_k, workspace=ws, workspace_bytes=nbytes)
    torch.cuda.synchronize()
    return dC.cpu().numpy(), nbytes


@pytest.mark.parametrize("layout", [(0, 0, 0), (1, 0, 1), (0, 1, 0), (1, 1, 1)], ids=lambda l: layout_name(*l))
@pytest.mark.parametrize("shape", [(2048, 2048, 256), (1664, 1920, 130), (2500, 1100, 96)], ids=lambda s: "x".join(map(str, s)))
def test_handover_schedule_is_the_single_chain(sgemm, orc, shape, layout):
    (M, N, K), (la, lb, lc) = shape, layout
    v = ws_variant(sgemm, la, lb, lc)
    A, B = orc.fill_ab(41, la, lb, M, N, K)
    got, nbytes = run_ex(sgemm, la, lb, lc, A, B, M, N, K, v, 1)
    assert nbytes > 0, "more tiles than SMs and a ragged last wave: the schedule must apply"
    plain, _ = run_ex(sgemm, la, lb, lc, A, B, M, N, K, v, 1, with_workspace=False)
    assert np.array_equal(bits(got), bits(plain))  # same bits as the round-robin schedule
    want = orc.sgemm_fma(lc, la, lb, A, B, M, N, K, threads=orc.max_threads())
    assert np.array_equal(bits(got), bits(want))   # which are the oracle's single chain
    assert sgemm.device_status() == 0


@pytest.mark.parametrize("layout", [(0, 0, 0), (1, 0, 1), (0, 1, 0), (1, 1, 1), (1, 0, 0)], ids=lambda l: layout_name(*l))
@pytest.mark.parametrize("shape", [(1024, 1024, 1024), (512, 768, 2048), (384, 200, 4100), (130, 70, 1000), (128, 128, 64)],
                         ids=lambda s: "x".join(map(str, s)))
def test_equal_ranges_schedule(sgemm, orc, shape, layout):
    (M, N, K), (la, lb, lc) = shape, layout
    v = ws_variant(sgemm, la, lb, lc)
    A, B = orc.fill_ab(43, la, lb, M, N, K)
    got, nbytes = run_ex(sgemm, la, lb, lc, A, B, M, N, K, v, -1)
    blk, offs, bnd = sgemm.stream_plan(lc, la, lb, M, N, K, v, -1, sms())
    if offs is None:
        # too little work to cut (fewer than 2 K tiles per extra CTA): the plain schedule, one chain
        assert nbytes == 0
        want = orc.sgemm_fma(lc, la, lb, A, B, M, N, K, threads=orc.max_threads())
    else:
        assert nbytes > 0 and len(bnd) > 0 and all(0 < b < K and b % blk[2] == 0 for b in bnd)
        want = orc.sgemm_fma_pieces(lc, la, lb, A, B, M, N, K, blk[0], blk[1], offs, bnd, threads=orc.max_threads())
    assert np.array_equal(bits(got), bits(want))
    ref = orc.sgemm_f64(lc, la, lb, A, B, M, N, K, threads=orc.max_threads())
    assert orc.error_metrics(lc, got, ref, M, N)["max_rel"] <= 1e-5 * math.sqrt(K)
    assert sgemm.device_status() == 0


def test_equal_ranges_identity_and_drop_in(sgemm, orc):
    """Identity B reproduces A bit for bit under any cut points; the drop-in entry takes the schedule from the table
    (the 1024^3 entries) and from its arena, call after call."""
    M = N = K = 1024
    A, _ = orc.fill_ab(1, 0, 0, M, N, K, with_b=False)
    dA, dI = torch.from_numpy(A).cuda(), torch.from_numpy(orc.fill_identity(0, K, N)).cuda()
    dC = torch.empty(M * N, dtype=torch.float32, device="cuda")
    p, _ = sgemm.select_config(M, N, K, 0, 0, 0)
    for _ in range(3):
        dC.fill_(float("nan"))
        sgemm.gemm(0, 0, 0, dC, dA, dI, M, N, K)
        torch.cuda.synchronize()
        assert torch.equal(dC.view(torch.int32), dA.view(torch.int32))
    A, B = orc.fill_ab(44, 0, 0, M, N, K)
    dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    first = None
    for _ in range(3):
        dC.fill_(float("nan"))
        sgemm.gemm(0, 0, 0, dC, dA, dB, M, N, K)
        torch.cuda.synchronize()
        got = dC.cpu().numpy()
        first = got if first is None else first
        assert np.array_equal(bits(got), bits(first))  # deterministic from call to call
    want = oracle_chain(sgemm, orc, 0, 0, 0, A, B, M, N, K, sms())
    assert np.array_equal(bits(first), bits(want))
    if p.split_k == 0:
        assert sgemm.stream_plan(0, 0, 0, M, N, K, -1, 0, sms())[1] is not None


def test_stream_plan_is_host_only(sgemm):
    """The cut points are plain integer arithmetic on (tiles, K tiles, CTAs): every tile's points are ascending
    multiples of block_k inside (0, K), and the pieces of all tiles together are CTAs - 1 + tiles (each CTA
    boundary that falls inside a tile adds one piece)."""
    v = ws_variant(sgemm)
    M, N, K = 1024, 1024, 16384
    blk, offs, bnd = sgemm.stream_plan(0, 0, 0, M, N, K, v, -1, 148)
    tiles = (M // blk[0]) * (N // blk[1])
    assert len(offs) == tiles + 1 and offs[0] == 0 and offs[-1] == len(bnd)
    for t in range(tiles):
        cuts = bnd[offs[t]:offs[t + 1]]
        assert all(0 < c < K and c % blk[2] == 0 for c in cuts) and list(cuts) == sorted(set(cuts))
    assert len(bnd) == 148 - 1 - sum(1 for c in range(1, 148) if (tiles * (K // blk[2]) * c // 148) % (K // blk[2]) == 0)
