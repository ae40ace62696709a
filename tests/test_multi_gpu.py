"""The sharded products on 2 GPUs, through the C ABI: one process per GPU (torch.distributed for the
plumbing) and, separately, a C++ caller with one thread per GPU.  Both exchange paths leave all of C
on every rank, bit-identical to the one-GPU product, and within the parity bounds of the CPU oracle;
the host-buffer path returns each rank's columns.  Skipped on boxes with fewer than two GPUs.  NVLS
is switched off for NCCL in the children; the fused path uses plain peer stores."""
import os
import socket
import subprocess
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
    from oracle import oracle_py as orc

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        pkg = entry.load_package()
        g = orc.Rng(1)  # the reference generator: same bytes on every rank
        a, b = g.randn((M, K), 0.0, K ** -0.5), g.randn((K, N), 0.0, K ** -0.5)
        A, B = torch.from_numpy(a).to(dev), torch.from_numpy(b).to(dev)
        # the one-GPU product without workspace, i.e. never K-split: the column blocks of the sharded call
        # (which never splits either) then add every element's terms in the same order
        whole = torch.empty((M, N), device=dev)
        pkg.gemm(A, B, whole, batch=1, M=M, N=N, K=K, lda=K, ldb=N, ldc=N)
        pkg.status()
        ok = {}
        if mode in ("fused", "nccl"):
            op = pkg.shard.ColumnShardedMatmul(M, N, K, rank=rank, world=world, device=dev, mode=mode)
            op.C.fill_(float("nan"))
            torch.cuda.synchronize()
            dist.barrier()
            # Calls back to back whose results DIFFER (A, 2A, A, ...), with a reader of C queued after each
            # on the same stream: the entry barrier of the next call must keep the peers' stores out
            # until that reader has run, or it would see a mix of C and 2C.
            A2 = 2.0 * A
            sums = []
            for it in range(4):
                C = op(A2 if it % 2 else A, B)
                sums.append(C.double().sum())
            C = op(A, B)
            torch.cuda.synchronize()
            dist.barrier()
            pkg.status()
            ok["bit_equal_to_one_gpu"] = bool(torch.equal(C, whole))
            want = [whole.double().sum(), (2.0 * whole).double().sum()]
            ok["reader_between_calls_saw_complete_c"] = bool(all(torch.equal(s, want[i % 2]) for i, s in enumerate(sums)))
            rows = np.arange(3, M, 41)
            ok["parity_vs_cpu_oracle"] = bool(
                orc.scaled_error(C.cpu().numpy()[rows], orc.matmul(a[rows], b)) <= orc.parity_tolerance(K))
        else:  # host buffers
            hop = pkg.shard.ShardedHostMatmul(M, N, K, rank=rank, world=world, device=dev, chunks=2)
            per, cols, col0 = hop.rows_per_rank, hop.cols, hop.col0
            h_a = torch.empty((per, K), dtype=torch.float32, pin_memory=True)
            h_b = torch.empty((K, cols), dtype=torch.float32, pin_memory=True)
            h_c = torch.empty((M, cols), dtype=torch.float32, pin_memory=True)
            h_a.copy_(torch.from_numpy(a[rank * per:(rank + 1) * per]))
            h_b.copy_(torch.from_numpy(np.ascontiguousarray(b[:, col0:col0 + cols])))
            for _ in range(2):
                h_c.fill_(float("nan"))
                hop(h_a.numpy(), h_b.numpy(), h_c.numpy())
            pkg.status()
            # A strip is a product of its own (fewer rows): the planner may split its K where the whole
            # product's is not split, so the columns agree to rounding, not bit for bit; a misplaced row or
            # chunk would be off by the size of the values.
            ok["own_columns_match_one_gpu"] = bool(
                orc.scaled_error(h_c.numpy(), whole[:, col0:col0 + cols].cpu().numpy()) <= 2e-6)
            rows = np.arange(1, M, 53)
            ok["parity_vs_cpu_oracle"] = bool(
                orc.scaled_error(h_c.numpy()[rows], orc.matmul(a[rows], np.ascontiguousarray(b[:, col0:col0 + cols])))
                <= orc.parity_tolerance(K))
        results[rank] = ok
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("shape", [(1024, 2048, 512), (768, 1000, 300)])  # even shards; ragged: 512 + 488 columns
@pytest.mark.parametrize("mode", ["nccl", "fused", "host"])
def test_two_gpu_column_shards(cuda, mode, shape):
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
        procs = [ctx.Process(target=_rank_main, args=(r, 2, port, mode, *shape, results)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=240)
        for p in procs:
            if p.is_alive():
                p.kill()
                pytest.fail("a rank did not finish")
            assert p.exitcode == 0
        got = dict(results)
        assert set(got) == {0, 1}
        for rank, ok in got.items():
            assert ok and all(ok.values()), (rank, ok)


def test_cpp_caller_two_gpus(cuda):
    """tests/cpp/test_shard_b200.cpp: a C++ program, one thread per GPU, runs the fused, the NCCL and
    the host-buffer sharded product through the C ABI and compares every rank's result with the
    unsharded product."""
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    exe = ROOT / "tests" / "cpp" / "test_shard_b200"
    if not exe.exists():
        import __graft_entry__ as entry

        entry.build()
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    proc = subprocess.run([str(exe)], capture_output=True, text=True, timeout=600, env=env)
    print(proc.stdout[-4000:])
    print(proc.stderr[-2000:])
    assert proc.returncode == 0, proc.stdout[-3000:]
    assert "ALL TESTS PASSED" in proc.stdout
