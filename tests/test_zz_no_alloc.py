"""b200_sgemm_splitk_static — the split-K entry point for hosts that may not allocate device memory
(a process whose own pool already owns the device, a latency-bound thread that must stay out of the
driver's allocator).  Its partial sums live in a fixed array inside the library's device image, so the call
reaches no allocation routine; this file checks, through the C ABI, that it computes exactly what the
workspace-taking entry computes, twice in a row on the shared array, that oversized requests are refused, and
that a call (after the first on the device, which makes the driver load the array) leaves the amount of free
device memory exactly as it found it.

Kept in a file that sorts last so that a run stopping at the first failure has already executed every
other test; it does not depend on any of them and also passes when run alone in a fresh process."""
import os
import subprocess
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _reference_result(sgemm, lc, la, lb, dA, dB, M, N, K, split):
    """The existing entry point with a caller-allocated workspace and the same split."""
    dC = torch.full((M * N,), float("nan"), dtype=torch.float32, device="cuda")
    nbytes = sgemm.workspace_bytes(lc, la, lb, M, N, K, -1, split)
    ws = torch.empty(max(nbytes, 1), dtype=torch.uint8, device="cuda")
    sgemm.gemm_ex(lc, la, lb, dC, dA, dB, M, N, K, split_k=split, workspace=ws, workspace_bytes=nbytes)
    torch.cuda.synchronize()
    return dC


def test_static_scratch_matches_workspace_entry_twice(sgemm, orc):
    # two calls in a row on the one shared array; the second is smaller and differently shaped, so stale
    # partial sums of the first lie right behind (and inside) the region it uses
    calls = [((0, 0, 0), (384, 256, 4096), 5, 21), ((1, 1, 1), (130, 70, 1000), 3, 22),
             ((0, 1, 0), (256, 192, 2048), 8, 23)]
    for (la, lb, lc), (M, N, K), split, seed in calls:
        A, B = orc.fill_ab(seed, la, lb, M, N, K)
        dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
        want = _reference_result(sgemm, lc, la, lb, dA, dB, M, N, K, split)
        got = torch.full((M * N,), float("nan"), dtype=torch.float32, device="cuda")
        sgemm.gemm_splitk_static(lc, la, lb, got, dA, dB, M, N, K, split)
        torch.cuda.synchronize()
        # the tolerance of the parity suite for equal summation order: none
        assert torch.equal(got.view(torch.int32), want.view(torch.int32)), ((la, lb, lc), (M, N, K), split)
        # and the result is the oracle's ordered split-K FMA chain
        p, _ = sgemm.select_config(M, N, K, lc, la, lb)
        chain = orc.sgemm_fma(lc, la, lb, A, B, M, N, K, splits=split, k_align=p.block_k, threads=orc.max_threads())
        assert np.array_equal(got.cpu().numpy().view(np.uint32), chain.view(np.uint32))
    assert sgemm.device_status() == 0


def test_static_scratch_limits(sgemm):
    import rocm_sgemm_b200 as pkg
    M = N = 2048
    K = 4096
    dA = torch.zeros(M * K, dtype=torch.float32, device="cuda")
    dB = torch.zeros(K * N, dtype=torch.float32, device="cuda")
    dC = torch.zeros(M * N, dtype=torch.float32, device="cuda")
    # 2 slices of 2048 x 2048 floats = 32 MiB: exactly the array, accepted
    assert 2 * M * N * 4 == pkg.STATIC_SCRATCH_BYTES
    sgemm.gemm_splitk_static(0, 0, 0, dC, dA, dB, M, N, K, 2)
    torch.cuda.synchronize()
    # 3 slices do not fit: refused with the dedicated status, nothing launched
    dC.fill_(7.0)
    with pytest.raises(pkg.SgemmError) as err:
        sgemm.gemm_splitk_static(0, 0, 0, dC, dA, dB, M, N, K, 3)
    assert err.value.status == pkg.SCRATCH_LIMIT
    assert "static scratch" in str(err.value)
    torch.cuda.synchronize()
    assert bool((dC == 7.0).all())
    # a split below 2 needs no scratch and is not this entry point's business
    with pytest.raises(pkg.SgemmError) as err:
        sgemm.gemm_splitk_static(0, 0, 0, dC, dA, dB, M, N, K, 1)
    assert err.value.status == pkg.INVALID_ARGUMENT


def test_a_call_leaves_free_device_memory_unchanged(sgemm):
    """The property in the entry point's name.  Everything torch needs is allocated first; one call has been made
    (it loads the array on the device); then free device memory as the driver reports it (cudaMemGetInfo) must be
    the same before and after further calls, which also exercise a new kernel shape each."""
    M, N, K = 512, 384, 2048
    dA = torch.rand(M * K, dtype=torch.float32, device="cuda")
    dB = torch.rand(K * N, dtype=torch.float32, device="cuda")
    dC = torch.empty(M * N, dtype=torch.float32, device="cuda")
    sgemm.gemm_splitk_static(0, 0, 0, dC, dA, dB, M, N, K, 4)  # first use at the latest: array and kernels loaded
    sgemm.gemm_splitk_static(0, 0, 0, dC, dA, dB, M, N, K, 2)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for split in (4, 2, 4):
        sgemm.gemm_splitk_static(0, 0, 0, dC, dA, dB, M, N, K, split)
    torch.cuda.synchronize()
    free_after = torch.cuda.mem_get_info()[0]
    assert free_after == free_before, f"free device memory changed by {free_before - free_after} bytes"


_FIRST_CALL_PROBE = r"""
import sys
sys.path.insert(0, sys.argv[1])
import torch
import rocm_sgemm_b200 as sg
M, N, K = 256, 256, 1024
dA = torch.rand(M * K, device="cuda"); dB = torch.rand(K * N, device="cuda"); dC = torch.empty(M * N, device="cuda")
ws = torch.empty(sg.workspace_bytes(0, 0, 0, M, N, K, -1, 2), dtype=torch.uint8, device="cuda")
# the same kernels through the workspace entry first, so that only the array's own module is new below
sg.gemm_ex(0, 0, 0, dC, dA, dB, M, N, K, split_k=2, workspace=ws, workspace_bytes=ws.numel())
torch.cuda.synchronize()
f0 = torch.cuda.mem_get_info()[0]
sg.gemm_splitk_static(0, 0, 0, dC, dA, dB, M, N, K, 2)
torch.cuda.synchronize()
f1 = torch.cuda.mem_get_info()[0]
sg.gemm_splitk_static(0, 0, 0, dC, dA, dB, M, N, K, 2)
torch.cuda.synchronize()
f2 = torch.cuda.mem_get_info()[0]
print("FIRST_CALL_DELTA", f0 - f1, "SECOND_CALL_DELTA", f1 - f2)
"""


def test_first_call_in_a_fresh_process_reserves_the_array_once():
    """What the documentation says about cost: in a fresh process (default module loading) the first call on a
    device is where the driver sets the 32 MiB array aside; the second call changes nothing.  With
    CUDA_MODULE_LOADING=EAGER in the environment the first delta is zero as well; both are accepted."""
    import rocm_sgemm_b200 as pkg
    r = subprocess.run([sys.executable, "-c", _FIRST_CALL_PROBE, ROOT], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    words = r.stdout.split()
    first, second = int(words[words.index("FIRST_CALL_DELTA") + 1]), int(words[words.index("SECOND_CALL_DELTA") + 1])
    print(f"first call reserved {first} bytes, second call {second} bytes")
    assert second == 0
    # nothing (already loaded) or the array plus the driver's rounding of the module's memory
    assert first == 0 or pkg.STATIC_SCRATCH_BYTES <= first <= pkg.STATIC_SCRATCH_BYTES + 16 * 1024 * 1024
