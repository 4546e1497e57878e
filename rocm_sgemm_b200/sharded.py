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


def a_upload_slice(layout_a: int, M: int, K: int, world: int, rank: int) -> tuple[int, int]:
    """(element offset, element count) of the part of the packed replicated A that `rank` uploads from host memory
    in the host-buffer pipeline: a 1/G-th contiguous range of the buffer (rows for row-major A, columns for col-major
    A), so that the all-gather of the ranges over NVLink rebuilds the whole of A on every GPU.  M*K must divide."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("bad rank / world size")
    if (M * K) % world:
        raise ValueError(f"A ({M}x{K}) does not divide into {world} equal ranges")
    n = M * K // world
    return rank * n, n


class ShardedHostGemm:
    """Column-sharded GEMM whose operands and result live in HOST memory, one object per rank.

    Every step each rank uploads 1/G of the replicated A and its own K x N/G slice of B over its own PCIe link,
    the ranks all-gather A over NVLink (NCCL), each multiplies (sg.gemm: the C ABI's drop-in entry) and downloads
    its M x N/G block of C.  Host traffic per step is (M*K + K*N + M*N) * 4 bytes for the whole job, whatever G is;
    uploading all of A on every rank would cost G times the A part.  Two steps are kept in flight on two streams
    with their own device buffers, so the copies of step i+1 run under the GEMM of step i.
    """

    def __init__(self, sg, layout_c: int, layout_a: int, layout_b: int, M: int, N: int, K: int, world: int, rank: int,
                 group=None):
        import torch
        self.sg, self.lc, self.la, self.lb = sg, layout_c, layout_a, layout_b
        self.M, self.N, self.K, self.world, self.rank, self.group = M, N, K, world, rank, group
        _, self.n = shard_columns(N, world, rank)
        self.a_off, self.a_len = a_upload_slice(layout_a, M, K, world, rank)
        self.slots = []
        for _ in range(2):
            self.slots.append({
                "stream": torch.cuda.Stream(),
                "A": torch.empty(M * K, dtype=torch.float32, device="cuda"),
                "B": torch.empty(K * self.n, dtype=torch.float32, device="cuda"),
                "C": torch.empty(M * self.n, dtype=torch.float32, device="cuda"),
                "done": None})
        self.h2d_bytes = (self.a_len + K * self.n) * 4
        self.d2h_bytes = M * self.n * 4
        self.step = 0

    def submit(self, hC_local, hA, hB_local):
        """Enqueues one step (pinned host tensors: the whole A, this rank's B slice, this rank's C block)."""
        import torch
        import torch.distributed as dist
        slot = self.slots[self.step % 2]
        self.step += 1
        if slot["done"] is not None:
            slot["done"].synchronize()  # the step that used these buffers two submits ago
        with torch.cuda.stream(slot["stream"]):
            mine = slot["A"][self.a_off:self.a_off + self.a_len]
            mine.copy_(hA[self.a_off:self.a_off + self.a_len], non_blocking=True)
            slot["B"].copy_(hB_local, non_blocking=True)
            if self.world > 1:
                dist.all_gather_into_tensor(slot["A"], mine, group=self.group)
            self.sg.gemm(self.lc, self.la, self.lb, slot["C"], slot["A"], slot["B"], self.M, self.n, self.K,
                         stream=slot["stream"])
            hC_local.copy_(slot["C"], non_blocking=True)
            slot["done"] = torch.cuda.Event()
            slot["done"].record(slot["stream"])
        return slot["done"]

    def wait_all(self):
        for slot in self.slots:
            if slot["done"] is not None:
                slot["done"].synchronize()


def block_offset(layout_c: int, M: int, N: int, world: int, rank: int) -> tuple[int, int]:
    """(element offset of rank's column block inside a full packed M x N matrix, leading dimension of that matrix).
    Row-major C: the block starts at column rank*N/G of row 0, rows are N apart.  Col-major C: the block is the
    contiguous range of its columns, columns are M apart."""
    n0, _ = shard_columns(N, world, rank)
    return (n0, N) if layout_c == ROW else (n0 * M, M)


class _DeviceArray:
    """Minimal __cuda_array_interface__ holder so that torch can view a raw device allocation."""

    def __init__(self, ptr: int, numel: int):
        self.__cuda_array_interface__ = {"shape": (numel,), "typestr": "<f4", "data": (int(ptr), False), "version": 3}


class PeerGatheredC:
    """A full-size C on every rank, each rank's copy mapped into all the other processes with CUDA IPC.

    With these mappings the GEMM's epilogue (b200_sgemm_multi) stores this rank's column block into every copy, so
    the all-gather that would follow the column-sharded product happens inside the kernel, over NVLink, tile by tile
    while the FMAs of the other tiles run.  Plain peer stores only (no multicast objects); every rank must pass a
    barrier after its kernel before anybody reads C, and before the buffers are closed.
    """

    def __init__(self, M: int, N: int, layout_c: int, world: int, rank: int, group=None):
        import torch.distributed as dist
        from cuda.bindings import runtime as rt
        self._rt, self.M, self.N, self.layout_c, self.world, self.rank = rt, M, N, layout_c, world, rank
        # Every step that can fail is followed by an exchange of its outcome, so that either all ranks end up with
        # a working object or all of them raise: nobody is left waiting in a collective for a rank that gave up.
        self.ptr, self.copies, why, mine = None, [], "", None
        err, ptr = rt.cudaMalloc(M * N * 4)
        if err == rt.cudaError_t.cudaSuccess:
            self.ptr = ptr
            err, handle = rt.cudaIpcGetMemHandle(self.ptr)
            if err == rt.cudaError_t.cudaSuccess:
                mine = bytes(handle.reserved)
            else:
                why = f"cudaIpcGetMemHandle failed: {err}"
        else:
            why = f"cudaMalloc failed: {err}"
        handles = [None] * world
        dist.all_gather_object(handles, mine, group=group)
        if any(h is None for h in handles):
            self._release()
            raise RuntimeError(why or "a peer could not export its copy of C")
        for g in range(world):
            if g == rank:
                self.copies.append(int(self.ptr))
                continue
            h = rt.cudaIpcMemHandle_t()
            h.reserved = handles[g]
            err, p = rt.cudaIpcOpenMemHandle(h, rt.cudaIpcMemLazyEnablePeerAccess)
            if err != rt.cudaError_t.cudaSuccess:
                why = f"cudaIpcOpenMemHandle failed for rank {g}: {err}"
                self.copies.append(0)
            else:
                self.copies.append(int(p))
        outcomes = [None] * world
        dist.all_gather_object(outcomes, why, group=group)
        if any(outcomes):
            self._release()
            raise RuntimeError(next(o for o in outcomes if o))

    def _release(self):
        """Closes the peer mappings and frees this rank's copy; no collective inside."""
        for g, p in enumerate(self.copies):
            if g != self.rank and p:
                self._rt.cudaIpcCloseMemHandle(p)
        self.copies = []
        if self.ptr is not None:
            self._rt.cudaFree(self.ptr)
            self.ptr = None

    def destinations(self) -> tuple[list[int], int]:
        """(addresses of this rank's column block in its own copy first, then in every peer's copy; leading dimension)."""
        off, ld = block_offset(self.layout_c, self.M, self.N, self.world, self.rank)
        order = [self.rank] + [g for g in range(self.world) if g != self.rank]
        return [self.copies[g] + 4 * off for g in order], ld

    def tensor(self):
        """This rank's full C as a 1-D torch tensor (a view of the raw allocation)."""
        import torch
        return torch.as_tensor(_DeviceArray(self.ptr, self.M * self.N), device="cuda")

    def close(self, group=None):
        import torch
        import torch.distributed as dist
        torch.cuda.synchronize()
        dist.barrier(group=group)  # nobody is still storing into a copy that is about to go away
        ptr, self.ptr = self.ptr, None
        self._release()            # peer mappings first ...
        dist.barrier(group=group)
        if ptr is not None:        # ... then the allocation they pointed into
            self._rt.cudaFree(ptr)


def fused_gather_gemm(sg, peer_c: PeerGatheredC, layout_c: int, layout_a: int, layout_b: int, A, B_local, M: int, N: int,
                      K: int, stream=None, variant: int = -1):
    """This rank's M x N/G product stored straight into every rank's full C (sg = the rocm_sgemm_b200 module)."""
    _, n = shard_columns(N, peer_c.world, peer_c.rank)
    dsts, ldc = peer_c.destinations()
    sg.gemm_multi(layout_c, layout_a, layout_b, dsts, A, B_local, M, n, K, ldc=ldc, variant=variant, stream=stream)
