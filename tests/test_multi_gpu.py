"""Column-sharded product on 2 GPUs (one process per GPU, NCCL over NVLink): both exchange
paths leave all of C on every rank, bit-identical to the one-GPU product.  Skipped on boxes with
fewer than two GPUs.  NVLS is switched off for NCCL in the children; the fused path uses plain
peer stores."""
import os
import socket
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _rank_main(rank, world, port, mode, M, N, K, results):
    import numpy as np
    import torch
    import torch.distributed as dist

    sys.path.insert(0, str(ROOT))
    import __graft_entry__ as entry

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        pkg = entry.load_package()
        gen = torch.Generator(device=dev).manual_seed(1)
        A = torch.randn((M, K), device=dev, generator=gen) / K ** 0.5
        B = torch.randn((K, N), device=dev, generator=gen) / K ** 0.5
        op = pkg.shard.ColumnShardedMatmul(M, N, K, rank=rank, world=world, device=dev, mode=mode)
        op.C.fill_(float("nan"))
        torch.cuda.synchronize()
        dist.barrier()
        for _ in range(2):
            C = op(A, B)
        torch.cuda.synchronize()
        dist.barrier()
        pkg.status()
        whole = pkg.matmul(A, B)
        pkg.status()
        results[rank] = bool(torch.equal(C, whole))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["nccl", "fused"])
def test_two_gpu_column_shards(cuda, mode):
    import torch
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        results = mgr.dict()
        procs = [ctx.Process(target=_rank_main, args=(r, 2, port, mode, 1024, 2048, 512, results)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=240)
        for p in procs:
            if p.is_alive():
                p.kill()
                pytest.fail("a rank did not finish")
            assert p.exitcode == 0
        assert dict(results) == {0: True, 1: True}
