"""N-column sharding of one large product over the GPUs of a node (one process per GPU).

Rank r holds all of A and computes columns ``[col0, col0 + cols)`` of ``C = A x B`` with the
single-GPU kernel working in place inside full-size row-major buffers (ldb = ldc = N).  Every
rank must end with all of C.  Two exchange paths:

``fused``   the kernel's epilogue stores each finished tile into its own C *and* into every
            peer's C (peer buffers mapped into this process through torch symmetric memory),
            so the gather rides under the remaining tiles' math and no separate collective
            runs.  Plain stores over NVLink; a barrier at the end orders completion.
``nccl``    compute the local columns, then one ``all_gather`` of the packed column blocks and
            a local unpack.  The baseline the fused path is measured against, and the only
            path that also runs on CPU tensors (gloo) for the host-logic tests.

The reference has nothing here to mirror (single device, src/cuda/runtime.cu:83).
"""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple

COL_ALIGN = 32  # shard boundaries fall on 128-byte column groups: TMA- and vector-store-legal


def column_shard(N: int, world: int, rank: int, align: int = COL_ALIGN) -> Tuple[int, int]:
    """Columns ``[col0, col0 + cols)`` owned by ``rank``: equal blocks rounded up to ``align``
    columns, the last rank taking what is left (possibly nothing when N is small)."""
    if world < 1 or not (0 <= rank < world) or N < 0:
        raise ValueError("bad shard request")
    per = -(-N // world)
    per = -(-per // align) * align
    col0 = min(N, rank * per)
    cols = min(N, col0 + per) - col0
    return col0, cols


def all_shards(N: int, world: int, align: int = COL_ALIGN) -> List[Tuple[int, int]]:
    return [column_shard(N, world, r, align) for r in range(world)]


def gather_columns(c_full, world: int, rank: int, group=None) -> None:
    """Completes ``c_full`` (M x N, this rank's columns already in place) with every peer's
    columns through one all_gather of packed blocks.  Works on CUDA (nccl) and CPU (gloo)."""
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


class ColumnShardedMatmul:
    """``C = A x B`` with B and C split by column blocks over the ranks of ``group``.

    ``compute_block(A, B, dests, col0, cols)`` computes the block into every buffer of
    ``dests``; the default calls the CUDA library.  Tests inject a CPU stand-in to exercise the
    sharding and gather logic without a GPU.
    """

    def __init__(self, M: int, N: int, K: int, *, rank: int, world: int, device, group=None,
                 mode: str = "fused", compute_block: Optional[Callable] = None):
        import torch

        if mode not in ("fused", "nccl"):
            raise ValueError("mode must be 'fused' or 'nccl'")
        self.M, self.N, self.K = M, N, K
        self.rank, self.world, self.group, self.mode = rank, world, group, mode
        self.device = torch.device(device)
        self.col0, self.cols = column_shard(N, world, rank)
        self._compute = compute_block or self._cuda_block
        self._handle = None
        self.peers = None
        if mode == "fused" and world > 1:
            import torch.distributed._symmetric_memory as symm

            self.C = symm.empty((M, N), dtype=torch.float32, device=self.device)
            grp = group if group is not None else torch.distributed.group.WORLD
            self._handle = symm.rendezvous(self.C, group=grp)
            # own buffer first, then the peers in ring order so that ranks do not all push to
            # the same destination at the same moment
            order = [(rank + i) % world for i in range(world)]
            self.peers = [self.C if r == rank else self._handle.get_buffer(r, (M, N), torch.float32)
                          for r in order]
        else:
            self.C = torch.empty((M, N), dtype=torch.float32, device=self.device)
            self.peers = [self.C]

    def _cuda_block(self, A, B, dests, col0, cols):
        from . import lib

        lib.gemm_colshard(A, B, dests, M=self.M, N=self.N, K=self.K, col0=col0, cols=cols,
                          lda=self.K, ldb=self.N, ldc=self.N)

    def barrier(self) -> None:
        import torch.distributed as dist

        if self.world == 1:
            return
        if self._handle is not None:
            self._handle.barrier()
        else:
            dist.barrier(group=self.group)

    def __call__(self, A, B):
        """Runs the sharded product; on return (after the stream's work and the closing
        barrier complete) ``self.C`` holds all of C on every rank."""
        if self.cols:
            dests = self.peers if self.mode == "fused" else [self.C]
            self._compute(A, B, dests, self.col0, self.cols)
        if self.world > 1:
            if self.mode == "fused":
                self.barrier()
            else:
                gather_columns(self.C, self.world, self.rank, self.group)
        return self.C
