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


def test_every_documented_option_is_accepted_and_the_list_is_complete(pkg):
    """The option names listed under b200_gemm_set_option in the header are exactly the ones the library
    accepts: each takes its default back, and a name the header does not list is refused."""
    import re
    from pathlib import Path

    header = (Path(__file__).resolve().parents[1] / "include" / "b200_gemm.h").read_text()
    block = header[: header.index("int b200_gemm_set_option(")]
    block = block[block.rindex("/*"):]
    documented = re.findall(r'^ \*   "([a-z_0-9]+)"', block, flags=re.M)
    defaults = {"pair_workers": 8, "pdl": 1, "map_cache": 1, "host_pipeline": 1, "tail_split": 1, "tf32_round": 1}
    lib = pkg.load()
    assert len(documented) >= 14 and len(set(documented)) == len(documented)
    for name in documented:
        assert lib.b200_gemm_set_option(name.encode(), defaults.get(name, 0)) == 0, name
    for name, bad in (("tile_n", 100), ("pair_mode", 3), ("head_mode", 2), ("block_k", 48), ("split_warps", 4),
                      ("pair_workers", 12), ("split_k", -1), ("group_m", -1)):
        assert name in documented
        assert lib.b200_gemm_set_option(name.encode(), bad) == -1, name


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


def test_plan_uses_the_deepest_split_the_workspace_holds(pkg):
    """b200_gemm_f32_plan without a device (148 SMs assumed): a workspace too small for the preferred
    K-split gives a shallower split, not an unsplit product; none gives none."""
    full = pkg.plan(1, 128, 256, 16384)
    assert full["split_k"] > 32 and full["workspace_used"] == pkg.workspace_bytes(1, 128, 256, 16384)
    small = pkg.plan(1, 128, 256, 16384, 4 << 20)
    assert 1 < small["split_k"] <= 32 and small["workspace_used"] <= 4 << 20 and small["kernels"] == 2
    assert small["workspace_used"] == small["split_k"] * 128 * 256 * 4
    none = pkg.plan(1, 128, 256, 16384, 0)
    assert none["split_k"] == 1 and none["kernels"] == 1 and none["workspace_used"] == 0
    one_part_only = pkg.plan(1, 128, 256, 16384, 128 * 256 * 4)  # room for one partial matrix: no split
    assert one_part_only["split_k"] == 1
    big = pkg.plan(1, 4096, 4096, 4096)
    assert big["pair"] == 1 and big["tile_n"] == 256 and big["tail_tiles"] > 0 and big["kernels"] == 3
    assert pkg.plan(1, 4096, 4096, 4096, 0)["kernels"] == 1
    narrow = pkg.plan(1, 50176, 8, 9)
    assert narrow["tile_n"] == 32 and narrow["split_k"] == 1
    with pytest.raises(pkg.B200Error):
        pkg.plan(1, 0, 8, 9)


def test_shard_arithmetic_of_the_library_matches_its_python_mirror(pkg):
    """b200_shard_columns / b200_shard_host_plan (what the CUDA path uses) against shard.py's
    column_shard / host_layout (what the gloo tests run on)."""
    shard = pkg.shard
    for N in (1, 31, 32, 33, 121, 4096, 16384, 16385):
        for world in (1, 2, 3, 4, 8):
            for rank in range(world):
                assert pkg.shard_columns(N, world, rank) == shard.column_shard(N, world, rank)
    for M, world, chunks in [(16384, 8, 0), (16384, 2, 8), (16384, 1, 0), (1024, 2, 0), (96, 3, 0), (8, 8, 0),
                             (4096, 4, 16)]:
        lay = pkg.shard_host_plan(M, world, chunks)
        assert (lay["chunks"], lay["rows_per_rank"], lay["chunk_rows"]) == shard.host_layout(M, world, chunks)
        assert lay["chunks"] * lay["chunk_rows"] * world == M
    for bad in [(100, 8, 0), (16384, 8, 17), (16384, 8, 3), (0, 2, 0)]:
        with pytest.raises(pkg.B200Error):
            pkg.shard_host_plan(*bad)
        with pytest.raises(ValueError):
            shard.host_layout(*bad)
    # the strips cover every row exactly once
    for M, world, chunks in [(64, 4, 4), (96, 3, 2)]:
        seen = np.zeros(M, np.int32)
        for ch in range(chunks):
            for first, count in shard.strip_global_rows(M, world, chunks, ch):
                seen[first:first + count] += 1
        assert (seen == 1).all()


def test_shard_comm_needs_a_device(pkg):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a device is present")
    with pytest.raises(pkg.B200Error):
        pkg.ShardComm(0, 2)


def _gloo_host_rank(rank, world, port, M, N, K, chunks, out_q):
    """A rank of the sharded host-buffer product, emulated on CPU: the chunk / strip / row arithmetic
    of b200_matmul_f32_host_sharded (through its Python mirror), the gather over gloo, the strip
    products by the CPU oracle."""
    import os

    import torch
    import torch.distributed as dist

    import __graft_entry__ as entry
    from oracle import oracle_py as orc

    pkg = entry.load_package()
    shard = pkg.shard
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = orc.Rng(8)
        a, b = g.randn((M, K)), g.randn((K, N))
        col0, cols = shard.column_shard(N, world, rank)
        chunks, per, cr = shard.host_layout(M, world, chunks)
        a_rows = np.ascontiguousarray(a[rank * per:(rank + 1) * per])       # what this rank's host holds
        b_cols = np.ascontiguousarray(b[:, col0:col0 + cols])
        c_cols = np.full((M, cols), np.nan, np.float32)
        for ch in range(chunks):
            mine = torch.from_numpy(np.ascontiguousarray(a_rows[ch * cr:(ch + 1) * cr]))
            parts = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(parts, mine)
            strip = torch.cat(parts, 0).numpy()                                # rank-major, like the device block
            block = orc.matmul(strip, b_cols) if cols else np.zeros((world * cr, 0), np.float32)
            for r, (first, count) in enumerate(shard.strip_global_rows(M, world, chunks, ch)):
                c_cols[first:first + count] = block[r * cr:(r + 1) * cr]
        want = orc.matmul(a, b)[:, col0:col0 + cols]
        out_q.put((rank, bool(np.array_equal(c_cols.view(np.uint32), want.view(np.uint32)))))
    finally:
        dist.destroy_process_group()


def test_sharded_host_layout_two_ranks_gloo():
    """world_size 2 on CPU: rows uploaded by halves, gathered chunk by chunk, multiplied by strips and
    scattered back — every rank ends with exactly its columns of the unsharded product."""
    import socket

    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_gloo_host_rank, args=(r, 2, port, 48, 70, 20, 4, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(results) == [(0, True), (1, True)]


def test_integration_doc_shows_the_seam_unit_that_is_compiled():
    """INTEGRATION.md prints oracle/seam/matmul_b200.cpp verbatim: the binding a maintainer is shown is
    the file `make -C oracle ref_cuda` compiles against the unmodified reference."""
    doc = (ROOT / "INTEGRATION.md").read_text()
    unit = (ROOT / "oracle" / "seam" / "matmul_b200.cpp").read_text()
    assert unit in doc
