"""CPU-only checks: the C-ABI library loads and exports every declared symbol, argument
errors are reported without a device, and the host-side shape / sharding logic mirrors the
reference's rules."""
import ctypes
import json
import re
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared_functions():
    text = (ROOT / "include" / "b200_gemm.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol(pkg):
    lib = pkg.load()
    names = declared_functions()
    assert len(names) >= 9
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/b200_gemm.h but not exported"
    assert set(pkg.lib.EXPORTS) == set(names)


def test_error_strings_and_options(pkg):
    lib = pkg.load()
    assert lib.b200_gemm_strerror(0) == b"success"
    assert b"invalid" in lib.b200_gemm_strerror(-1)
    assert lib.b200_gemm_strerror(-5)
    assert lib.b200_gemm_set_option(b"no_such_option", 1) == -1
    assert lib.b200_gemm_set_option(b"tile_n", 48) == -1
    assert lib.b200_gemm_set_option(b"tile_n", 0) == 0
    assert lib.b200_gemm_set_option(None, 0) == -1
    assert lib.b200_gemm_launch_count() >= 0


def test_no_cpu_fallback_without_device(pkg):
    """Without a CUDA device the entry points fail loudly instead of computing elsewhere."""
    import torch

    if torch.cuda.is_available():
        pytest.skip("a device is present")
    a = np.ones((4, 4), np.float32)
    out = np.zeros((4, 4), np.float32)
    with pytest.raises(pkg.B200Error):
        pkg.matmul_host(a, a, out, batch=1, rows=4, inner=4, cols=4, a_batched=False, b_batched=False)
    assert not out.any()
    with pytest.raises(RuntimeError):
        pkg.matmul(torch.ones(4, 4), torch.ones(4, 4))


def test_shape_rules_mirror_the_reference(pkg, golden_dir):
    """src/tensor_ops.cpp:476-503: the same combinations throw, the same batch plan results."""
    plan = pkg.engine._batch_plan
    spec = json.loads((golden_dir / "known_answers.json").read_text())
    for case in spec["throws"]:
        with pytest.raises(ValueError):
            plan(case["a_shape"], case["b_shape"])
    assert plan((2, 3), (3, 2)) == ([], 1, 2, 3, 2, False, False)
    assert plan((4, 3, 17, 23), (4, 3, 23, 11)) == ([4, 3], 12, 17, 23, 11, True, True)
    assert plan((8, 12, 40), (40, 20)) == ([8], 8, 12, 40, 20, True, False)
    assert plan((12, 40), (8, 40, 20)) == ([8], 8, 12, 40, 20, False, True)


def test_column_shards_cover_n_exactly(pkg):
    shard = pkg.shard
    for N in (0, 1, 31, 32, 33, 121, 4096, 16384, 16385):
        for world in (1, 2, 3, 4, 8):
            blocks = shard.all_shards(N, world)
            assert blocks[0][0] == 0
            pos = 0
            for col0, cols in blocks:
                assert cols >= 0 and (cols == 0 or col0 == pos)
                assert col0 % shard.COL_ALIGN == 0 or cols == 0
                pos += cols
            assert pos == N
    assert shard.all_shards(16384, 8) == [(i * 2048, 2048) for i in range(8)]
    with pytest.raises(ValueError):
        shard.column_shard(10, 2, 2)


def _gloo_rank(rank, world, port, M, N, K, out_q):
    import os
    import sys

    import torch
    import torch.distributed as dist

    sys.path.insert(0, str(ROOT))
    import __graft_entry__ as entry
    from oracle import oracle_py as orc

    pkg = entry.load_package()
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = orc.Rng(5)
        a, b = g.randn((M, K)), g.randn((K, N))

        def cpu_block(A, B, dests, col0, cols):  # stand-in for the CUDA kernel: same contract
            block = orc.matmul(A.numpy(), np.ascontiguousarray(B.numpy()[:, col0:col0 + cols]))
            for d in dests:
                d[:, col0:col0 + cols] = torch.from_numpy(block)

        op = pkg.shard.ColumnShardedMatmul(M, N, K, rank=rank, world=world, device="cpu", mode="nccl",
                                           compute_block=cpu_block)
        op.C.fill_(float("nan"))
        c = op(torch.from_numpy(a), torch.from_numpy(b)).numpy()
        want = orc.matmul(a, b)
        out_q.put((rank, bool(np.array_equal(c.view(np.uint32), want.view(np.uint32)))))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("N", [96, 130])
def test_sharded_gather_two_ranks_gloo(N):
    """world_size 2 on CPU: every rank ends with the whole product, bit-identical to the
    unsharded one (a column block is computed with the same per-row k order)."""
    import socket

    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_gloo_rank, args=(r, 2, port, 40, N, 24, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(results) == [(0, True), (1, True)]
