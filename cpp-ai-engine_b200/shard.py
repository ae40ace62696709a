"""N-column sharding of one large product over the GPUs of a node (one process per GPU).

Rank r holds all of A and computes columns ``[col0, col0 + cols)`` of ``C = A x B`` with the
single-GPU kernel working in place inside full-size row-major buffers (ldb = ldc = N).  Every
rank must end with all of C.  The product path is the library's ``b200_gemm_f32_sharded`` behind a
``b200_shard_comm`` handle; this module only supplies what the handle needs from
``torch.distributed`` (the peers' buffers through symmetric memory, or the NCCL communicator):

``fused``   [entry barrier] [product kernel whose forwarder warps store every finished tile into
            every peer's C over NVLink] [exit barrier], all inside the library call.
``nccl``    local columns, one ``ncclAllGather`` of packed column blocks, copies into C.

:class:`ShardedHostMatmul` is the same product from host buffers (``b200_matmul_f32_host_sharded``):
every rank uploads 1/world of A's rows and its own columns of B, the rows are all-gathered over
NVLink chunk by chunk, and the own columns of C go back to the host.

Host-logic tests (gloo ranks on CPU) inject ``compute_block`` and run the Python gather below on
CPU tensors; nothing on the CUDA path goes through it.

The reference has nothing here to mirror (single device, src/cuda/runtime.cu:83).
"""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple

COL_ALIGN = 32  # shard boundaries fall on 128-byte column groups: TMA- and vector-store-legal


def column_shard(N: int, world: int, rank: int, align: int = COL_ALIGN) -> Tuple[int, int]:
    """Columns ``[col0, col0 + cols)`` owned by ``rank``: equal blocks rounded up to ``align``
    columns, the last rank taking what is left (possibly nothing when N is small).  Mirror of
    ``b200_shard_columns`` (the CPU tests hold the two together)."""
    if world < 1 or not (0 <= rank < world) or N < 0:
        raise ValueError("bad shard request")
    per = -(-N // world)
    per = -(-per // align) * align
    col0 = min(N, rank * per)
    cols = min(N, col0 + per) - col0
    return col0, cols


def all_shards(N: int, world: int, align: int = COL_ALIGN) -> List[Tuple[int, int]]:
    return [column_shard(N, world, r, align) for r in range(world)]


def host_layout(M: int, world: int, chunks: int = 0) -> Tuple[int, int, int]:
    """``(chunks, rows_per_rank, chunk_rows)`` of the sharded host-buffer product — mirror of
    ``b200_shard_host_plan``.  Rank r keeps rows ``[r * rows_per_rank, (r + 1) * rows_per_rank)`` of A
    and uploads them in ``chunks`` pieces."""
    if M <= 0 or world < 1 or M % world or chunks > 16:
        raise ValueError("M must be a positive multiple of the number of ranks; at most 16 chunks")
    per = M // world
    if chunks <= 0:
        chunks = 4 if (per % 4 == 0 and per >= 512) else 2 if (per % 2 == 0 and per >= 256) else 1
    if per % chunks:
        raise ValueError("the rows of a rank do not divide into that many chunks")
    return chunks, per, per // chunks


def strip_global_rows(M: int, world: int, chunks: int, chunk: int) -> List[Tuple[int, int]]:
    """The global row ranges ``(first, count)`` that make up strip ``chunk`` of the sharded host
    product, in the order they lie in the gathered block (rank-major)."""
    chunks, per, cr = host_layout(M, world, chunks)
    return [(r * per + chunk * cr, cr) for r in range(world)]


def gather_columns(c_full, world: int, rank: int, group=None) -> None:
    """Completes ``c_full`` (M x N, this rank's columns already in place) with every peer's
    columns through one all_gather of packed blocks.  Used by the host-logic tests on CPU (gloo);
    the CUDA path gathers inside ``b200_gemm_f32_sharded``."""
    import torch
    import torch.distributed as dist

    M, N = c_full.shape
    shards = all_shards(N, world)
    width = max(c for _, c in shards)
    if width == 0:
        return
    packed = torch.zeros((M, width), dtype=c_full.dtype, device=c_full.device)
    col0, cols = shards[rank]
    if cols:
        packed[:, :cols].copy_(c_full[:, col0:col0 + cols])
    gathered = torch.empty((world, M, width), dtype=c_full.dtype, device=c_full.device)
    dist.all_gather_into_tensor(gathered.view(-1), packed.view(-1), group=group) \
        if c_full.is_cuda else dist.all_gather(list(gathered.unbind(0)), packed, group=group)
    for r, (r0, rc) in enumerate(shards):
        if r != rank and rc:
            c_full[:, r0:r0 + rc].copy_(gathered[r, :, :rc])


def _nccl_comm_ptr(device, group=None) -> int:
    """The ``ncclComm_t`` of ``group`` on ``device`` as an integer (created if it does not exist yet)."""
    import torch
    import torch.distributed as dist

    grp = group if group is not None else dist.group.WORLD
    backend = grp._get_backend(torch.device(device))
    if not hasattr(backend, "_comm_ptr"):
        raise RuntimeError("this torch build does not expose the NCCL communicator (ProcessGroupNCCL._comm_ptr)")
    warm = torch.zeros(1, device=device)
    dist.all_reduce(warm, group=grp)  # makes sure the communicator exists
    torch.cuda.synchronize(device)
    return int(backend._comm_ptr())


class ColumnShardedMatmul:
    """``C = A x B`` with B and C split by column blocks over the ranks of ``group``.

    On CUDA the call is ``b200_gemm_f32_sharded`` (``mode`` "fused" or "nccl").  With
    ``compute_block(A, B, dests, col0, cols)`` injected — the host-logic tests do that, on CPU
    tensors over gloo — the block is computed by that stand-in and gathered by :func:`gather_columns`.
    """

    def __init__(self, M: int, N: int, K: int, *, rank: int, world: int, device, group=None,
                 mode: str = "fused", compute_block: Optional[Callable] = None, precision: int = 0):
        import torch

        if mode not in ("fused", "nccl"):
            raise ValueError("mode must be 'fused' or 'nccl'")
        self.M, self.N, self.K = M, N, K
        self.rank, self.world, self.group, self.mode = rank, world, group, mode
        self.device = torch.device(device)
        self.precision = precision
        self.col0, self.cols = column_shard(N, world, rank)
        self._compute = compute_block
        self._comm = None
        self._handles = []
        if compute_block is not None:  # test seam: no library, no GPU
            self.C = torch.empty((M, N), dtype=torch.float32, device=self.device)
            return
        from . import lib

        self._comm = lib.ShardComm(rank, world)
        if mode == "fused" and world > 1:
            import torch.distributed._symmetric_memory as symm

            grp = group if group is not None else torch.distributed.group.WORLD
            self.C = symm.empty((M, N), dtype=torch.float32, device=self.device)
            self._flags = symm.empty((64,), dtype=torch.int32, device=self.device)
            self._flags.zero_()
            torch.cuda.synchronize(self.device)
            hc = symm.rendezvous(self.C, group=grp)
            hf = symm.rendezvous(self._flags, group=grp)
            hf.barrier()  # every rank's flag block is zero before anybody can signal
            torch.cuda.synchronize(self.device)
            self._handles = [hc, hf]
            c_bufs = [self.C if r == rank else hc.get_buffer(r, (M, N), torch.float32) for r in range(world)]
            flags = [self._flags if r == rank else hf.get_buffer(r, (64,), torch.int32) for r in range(world)]
            self._peer_views = (c_bufs, flags)  # keep the mappings alive
            self._comm.set_peers(c_bufs, flags)
        else:
            self.C = torch.empty((M, N), dtype=torch.float32, device=self.device)
            if world > 1:
                self._comm.set_nccl(_nccl_comm_ptr(self.device, group))

    def __call__(self, A, B):
        """Runs the sharded product; once the stream's work has completed, ``self.C`` holds all of C
        on every rank."""
        if self._comm is not None:
            from . import lib

            lib.gemm_sharded(self._comm, lib.SHARD_FUSED if self.mode == "fused" else lib.SHARD_NCCL, A, B, self.C,
                             M=self.M, N=self.N, K=self.K, lda=self.K, ldb=self.N, ldc=self.N,
                             precision=self.precision)
            return self.C
        if self.cols:
            self._compute(A, B, [self.C], self.col0, self.cols)
        if self.world > 1:
            gather_columns(self.C, self.world, self.rank, self.group)
        return self.C


class ShardedHostMatmul:
    """The sharded product from HOST buffers through ``b200_matmul_f32_host_sharded``.

    ``a_rows``: this rank's rows of A, ``(M / world, K)``; ``b_cols``: its columns of B packed,
    ``(K, cols)``; ``c_cols``: receives its columns of C, ``(M, cols)`` — numpy float32 arrays, best
    page-locked (``torch.empty(..., pin_memory=True).numpy()``)."""

    def __init__(self, M: int, N: int, K: int, *, rank: int, world: int, device, group=None, chunks: int = 0):
        from . import lib

        self.M, self.N, self.K, self.rank, self.world = M, N, K, rank, world
        self.col0, self.cols = column_shard(N, world, rank)
        self.chunks, self.rows_per_rank, self.chunk_rows = host_layout(M, world, chunks)
        self._comm = lib.ShardComm(rank, world)
        if world > 1:
            self._comm.set_nccl(_nccl_comm_ptr(device, group))

    def __call__(self, a_rows, b_cols, c_cols) -> None:
        from . import lib

        if a_rows.shape != (self.rows_per_rank, self.K) or b_cols.shape != (self.K, max(self.cols, 0)) \
                or c_cols.shape != (self.M, max(self.cols, 0)):
            raise ValueError("host buffers do not have the shapes of this rank's shard")
        lib.matmul_host_sharded(self._comm, a_rows, b_cols, c_cols, M=self.M, N=self.N, K=self.K,
                                chunks=self.chunks)
