"""Column-sharded product with the all-gather folded into the GEMM epilogue (peer stores over NVLink).

Needs two GPUs: one process per GPU, C copies mapped across processes with CUDA IPC
(rocm_sgemm_b200.sharded.PeerGatheredC), every rank's kernel stores its column block into every copy.
The result on every rank must equal, bit for bit, what the ranks' separate products assemble to.
Skipped on a single-GPU box; the multi-destination store itself is covered on one GPU by
tests/test_blas_batched.py::test_multi_destination_store.
"""
import os
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank: int, world: int, port: int, layout_c: int, out):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    import oracle
    import rocm_sgemm_b200 as sg
    from rocm_sgemm_b200 import sharded

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        M, N, K = 512, 1024, 256
        la, lb = 0, 0
        A, B = oracle.fill_ab(60, la, lb, M, N, K)
        dA = torch.from_numpy(A).cuda()
        dB = sharded.local_b_slice(torch.from_numpy(B).cuda(), lb, K, N, world, rank)
        pc = sharded.PeerGatheredC(M, N, layout_c, world, rank)
        pc.tensor().fill_(float("nan"))
        torch.cuda.synchronize()
        dist.barrier()
        sharded.fused_gather_gemm(sg, pc, layout_c, la, lb, dA, dB, M, N, K)
        torch.cuda.synchronize()
        dist.barrier()  # every rank's stores have landed
        got = pc.tensor().cpu().numpy().copy()
        want = oracle.sgemm_fma(layout_c, la, lb, A, B, M, N, K, splits=1, threads=oracle.max_threads())
        ok = bool(np.array_equal(got.view(np.uint32), want.view(np.uint32)))
        status = sg.device_status()
        pc.close()
        out.put((rank, ok, status))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("layout_c", [0, 1], ids=["Crow", "Ccol"])
def test_fused_gather_two_gpus(layout_c):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    world, port = 2, 29620 + layout_c
    procs = [ctx.Process(target=_worker, args=(r, world, port, layout_c, out)) for r in range(world)]
    for p in procs:
        p.start()
    results = []
    for _ in range(world):
        results.append(out.get(timeout=240))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(r[0] for r in results) == [0, 1]
    assert all(ok for _, ok, _ in results), results
    assert all(st == 0 for _, _, st in results), results
