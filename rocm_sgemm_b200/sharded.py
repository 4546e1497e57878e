"""Column-sharded GEMM over several GPUs of one box (one process per GPU).

C is partitioned by N-column blocks: rank g of G owns columns [g*N/G, (g+1)*N/G), holds all of A and
its K x N/G slice of B, and computes an M x N/G GEMM with no communication.  Afterwards the blocks can
be all-gathered (NCCL over NVLink) into a full C on every rank.  The reference has no multi-GPU code;
this is the driver its single-GPU operator is embedded in.

Everything here is layout bookkeeping on torch tensors (CPU or CUDA); the GEMM itself is passed in.
"""
from __future__ import annotations

ROW, COL = 0, 1


def shard_columns(N: int, world: int, rank: int) -> tuple[int, int]:
    """(first column, number of columns) of rank's block; N must divide evenly."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("bad rank / world size")
    if N % world:
        raise ValueError(f"N={N} does not divide over {world} ranks")
    n = N // world
    return rank * n, n


def local_b_slice(B, layout_b: int, K: int, N: int, world: int, rank: int):
    """Packed K x N/G slice of a packed K x N matrix B (1-D tensor) in the same layout.
    Row-major B: a strided column block made contiguous; col-major B: a contiguous range."""
    n0, n = shard_columns(N, world, rank)
    if layout_b == ROW:
        return B.view(K, N)[:, n0:n0 + n].contiguous().view(-1)
    return B.view(N, K)[n0:n0 + n].contiguous().view(-1)


def assemble_c(blocks, layout_c: int, M: int, N: int, world: int):
    """Full packed M x N matrix from the concatenation of the ranks' packed M x N/G blocks
    (what all_gather_into_tensor returns).  Col-major C: the concatenation already is the matrix.
    Row-major C: [G][M][N/G] -> [M][G][N/G]."""
    n = N // world
    if layout_c == COL:
        return blocks.view(-1)
    return blocks.view(world, M, n).permute(1, 0, 2).contiguous().view(-1)


def sharded_gemm(gemm, layout_c: int, layout_a: int, layout_b: int, C_local, A, B_local, M: int, N: int, K: int,
                 world: int, rank: int, **kw):
    """Runs gemm(layout_c, layout_a, layout_b, C_local, A, B_local, M, N/G, K, **kw) for this rank."""
    _, n = shard_columns(N, world, rank)
    return gemm(layout_c, layout_a, layout_b, C_local, A, B_local, M, n, K, **kw)


def all_gather_c(C_local, layout_c: int, M: int, N: int, world: int, group=None):
    """All-gather of the C blocks (torch.distributed; NCCL on GPUs) and assembly into the full matrix."""
    import torch
    import torch.distributed as dist
    full = torch.empty(world * C_local.numel(), dtype=C_local.dtype, device=C_local.device)
    dist.all_gather_into_tensor(full, C_local, group=group)
    return assemble_c(full, layout_c, M, N, world)
