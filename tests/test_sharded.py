"""Column sharding over ranks: slice arithmetic, gather layout, and a world-size-2 run over gloo on CPU
(the local GEMM is the oracle there: the subject is the sharding logic, not a kernel)."""
import os
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")

from common import LAYOUTS, as2d, bits  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_columns():
    from rocm_sgemm_b200 import sharded
    assert sharded.shard_columns(16384, 8, 3) == (6144, 2048)
    assert sharded.shard_columns(8, 1, 0) == (0, 8)
    with pytest.raises(ValueError):
        sharded.shard_columns(10, 4, 0)
    with pytest.raises(ValueError):
        sharded.shard_columns(8, 2, 2)


@pytest.mark.parametrize("world", [1, 2, 4])
def test_slices_and_assembly_roundtrip(orc, world):
    from rocm_sgemm_b200 import sharded
    M, N, K = 12, 16, 20
    for (la, lb, lc) in LAYOUTS:
        A, B = orc.fill_ab(3, la, lb, M, N, K)
        full = orc.sgemm_fma(lc, la, lb, A, B, M, N, K)
        blocks = []
        for r in range(world):
            Bl = sharded.local_b_slice(torch.from_numpy(B), lb, K, N, world, r).numpy()
            n0, n = sharded.shard_columns(N, world, r)
            # the slice is the packed K x n sub-matrix
            assert np.array_equal(as2d(Bl, lb, K, n), as2d(B, lb, K, N)[:, n0:n0 + n])
            blocks.append(orc.sgemm_fma(lc, la, lb, A, np.ascontiguousarray(Bl), M, n, K))
        got = sharded.assemble_c(torch.from_numpy(np.concatenate(blocks)), lc, M, N, world).numpy()
        assert np.array_equal(bits(got), bits(full)), (la, lb, lc)


def _worker(rank, world, port, results):
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    import oracle
    from rocm_sgemm_b200 import sharded
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, N, K = 24, 32, 40
        ok = True
        for (la, lb, lc) in [(0, 0, 0), (1, 1, 1), (0, 1, 0), (1, 0, 1)]:
            A, B = oracle.fill_ab(4, la, lb, M, N, K)
            Bl = sharded.local_b_slice(torch.from_numpy(B), lb, K, N, world, rank)
            _, n = sharded.shard_columns(N, world, rank)
            Cl = torch.empty(M * n, dtype=torch.float32)

            def gemm(lc_, la_, lb_, C_, A_, B_, M_, N_, K_):
                C_.copy_(torch.from_numpy(oracle.sgemm_fma(lc_, la_, lb_, A_.numpy(), B_.numpy(), M_, N_, K_)))

            # the host pipeline's upload rule: each rank holds 1/G of the packed A, an in-place all-gather rebuilds it
            off, cnt = sharded.a_upload_slice(la, M, K, world, rank)
            dA = torch.zeros(M * K, dtype=torch.float32)
            dA[off:off + cnt] = torch.from_numpy(A)[off:off + cnt]
            parts = [torch.empty(cnt, dtype=torch.float32) for _ in range(world)]
            dist.all_gather(parts, dA[off:off + cnt].clone())
            ok = ok and np.array_equal(torch.cat(parts).numpy().view(np.uint32), A.view(np.uint32))
            sharded.sharded_gemm(gemm, lc, la, lb, Cl, torch.from_numpy(A), Bl, M, N, K, world, rank)
            full = sharded.all_gather_c(Cl, lc, M, N, world).numpy()
            want = oracle.sgemm_fma(lc, la, lb, A, B, M, N, K)
            ok = ok and np.array_equal(full.view(np.uint32), want.view(np.uint32))
        results[rank] = ok
    finally:
        dist.destroy_process_group()


def test_two_ranks_over_gloo():
    import torch.multiprocessing as mp
    world = 2
    port = 29500 + (os.getpid() % 1000)
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
    assert dict(results) == {0: True, 1: True}


def test_block_offset_matches_assembly():
    """The offset / leading dimension that the fused epilogue stores with addresses the same elements as the
    assembly of gathered blocks."""
    import torch
    from rocm_sgemm_b200 import sharded
    M, N, world = 6, 8, 4
    n = N // world
    for lc in (0, 1):
        full = torch.full((M * N,), -1.0)
        blocks = []
        for r in range(world):
            blk = torch.arange(M * n, dtype=torch.float32) + 1000 * r
            blocks.append(blk)
            off, ld = sharded.block_offset(lc, M, N, world, r)
            view = blk.view(M, n) if lc == 0 else blk.view(n, M)
            for o in range(view.shape[0]):
                full[off + o * ld: off + o * ld + view.shape[1]] = view[o]
        want = sharded.assemble_c(torch.cat(blocks), lc, M, N, world)
        assert torch.equal(full, want)


def test_a_upload_slices_tile_the_operand():
    from rocm_sgemm_b200 import sharded
    M, K = 16, 24
    for world in (1, 2, 4, 8):
        seen = np.zeros(M * K, dtype=np.int32)
        for r in range(world):
            off, cnt = sharded.a_upload_slice(0, M, K, world, r)
            assert cnt == M * K // world
            seen[off:off + cnt] += 1
        assert (seen == 1).all()
    with pytest.raises(ValueError):
        sharded.a_upload_slice(0, 3, 5, 2, 0)
    with pytest.raises(ValueError):
        sharded.a_upload_slice(0, 4, 4, 2, 2)
