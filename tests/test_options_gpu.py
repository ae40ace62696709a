"""The tuning options that select other code paths of the same product (b200_gemm_set_option): every
variant must give the default path's result — bit for bit where the summation order is the same, within
the parity bound where it is not — and exact results on small integers."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def dev(x, cuda):
    import torch

    return torch.from_numpy(np.ascontiguousarray(x)).to(cuda)


def product(pkg, cuda, A, B, M, N, K, **kw):
    import torch

    ws_bytes = pkg.workspace_bytes(1, M, N, K)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=cuda)
    C = torch.full((M, N), float("nan"), device=cuda)
    pkg.gemm(A, B, C, batch=1, M=M, N=N, K=K, ldc=N, workspace=ws, workspace_bytes=ws_bytes, **kw)
    pkg.status()
    return C


@pytest.mark.parametrize("option,value,default", [("pair_workers", 16, 8), ("split_warps", 8, 0)])
def test_pair_kernel_warp_layouts_are_bit_identical(pkg, orc, cuda, option, value, default):
    """pair_workers = 16: half the accumulators per thread, twice the warps.  split_warps = 8: eight more
    warps that only split the stages while the eight workers only drain and store.  The same sums in the
    same order either way."""
    import torch

    g = orc.Rng(70)
    for M, N, K in ((2048, 2048, 512), (4000, 4100, 256)):  # whole and ragged 256 x 256 tiles
        a, b = g.randn((M, K)), g.randn((K, N))
        A, B = dev(a, cuda), dev(b, cuda)
        want = product(pkg, cuda, A, B, M, N, K, lda=K, ldb=N)
        assert pkg.plan(1, M, N, K)["pair"] == 1, "expected the CTA-pair kernel for this shape"
        pkg.set_option(option, value)
        try:
            got = product(pkg, cuda, A, B, M, N, K, lda=K, ldb=N)
        finally:
            pkg.set_option(option, default)
        assert torch.equal(got, want)
        rows = np.arange(0, M, 29)
        assert orc.scaled_error(got.cpu().numpy()[rows], orc.matmul(a[rows], b)) <= orc.parity_tolerance(K)


@pytest.mark.parametrize("form", ["NN", "NT", "TN", "TT"])
def test_k_blocks_of_64_match_the_default_and_are_exact_on_integers(pkg, orc, cuda, form):
    """block_k = 64 (narrow tiles, TMA loader): two swizzle rows of k per pipeline stage."""
    tA, tB = form[0] == "T", form[1] == "T"
    g = orc.Rng(71)
    for M, N, K in ((300, 96, 384), (130, 61, 200), (64, 40, 96)):
        a = g.randn((K, M) if tA else (M, K))
        b = g.randn((N, K) if tB else (K, N))
        ai = (np.arange(a.size).reshape(a.shape) % 9 - 4).astype(np.float32)
        bi = (np.arange(b.size).reshape(b.shape) % 7 - 3).astype(np.float32)
        kw = dict(transA=tA, transB=tB, lda=a.shape[1], ldb=b.shape[1])
        pkg.set_option("block_k", 64)
        try:
            got = product(pkg, cuda, dev(a, cuda), dev(b, cuda), M, N, K, **kw).cpu().numpy()
            exact = product(pkg, cuda, dev(ai, cuda), dev(bi, cuda), M, N, K, **kw).cpu().numpy()
        finally:
            pkg.set_option("block_k", 0)
        opa, opb = (a.T if tA else a), (b.T if tB else b)
        want = orc.matmul(np.ascontiguousarray(opa), np.ascontiguousarray(opb))
        assert orc.scaled_error(got, want) <= orc.parity_tolerance(K)
        orc.assert_no_further_from_fp64(got, want, opa.astype(np.float64) @ opb.astype(np.float64), factor=1.5)
        assert np.array_equal(exact, (ai.T if tA else ai) @ (bi.T if tB else bi))


def test_truncated_head_mode_stays_within_parity(pkg, orc, cuda):
    """head_mode = 1: the tensor core's truncation of the raw tile is the head, only the tail is written;
    1.3-1.4x the default's error against fp64, far inside the bound against the CPU loop; exact on integers."""
    g = orc.Rng(72)
    M, N, K = 512, 512, 512
    a, b = g.rand((M, K), -1, 1), g.rand((K, N), -1, 1)
    ai = (np.arange(M * K).reshape(M, K) % 5 - 2).astype(np.float32)
    bi = (np.arange(K * N).reshape(K, N) % 3 - 1).astype(np.float32)
    pkg.set_option("head_mode", 1)
    try:
        got = product(pkg, cuda, dev(a, cuda), dev(b, cuda), M, N, K, lda=K, ldb=N).cpu().numpy()
        exact = product(pkg, cuda, dev(ai, cuda), dev(bi, cuda), M, N, K, lda=K, ldb=N).cpu().numpy()
    finally:
        pkg.set_option("head_mode", 0)
    want = orc.matmul(a, b)
    assert orc.scaled_error(got, want) <= orc.parity_tolerance(K)
    orc.assert_no_further_from_fp64(got, want, a.astype(np.float64) @ b.astype(np.float64))
    assert np.array_equal(exact, ai @ bi)


def test_plain_launches_and_fresh_tensor_maps_give_the_same_bits(pkg, orc, cuda):
    """pdl = 0 (no programmatic dependent launch) and map_cache = 0 change how a product is launched, not
    what it computes."""
    import torch

    g = orc.Rng(73)
    M, N, K = 777, 300, 260
    A, B = dev(g.randn((M, K)), cuda), dev(g.randn((K, N)), cuda)
    want = product(pkg, cuda, A, B, M, N, K, lda=K, ldb=N)
    for name in ("pdl", "map_cache"):
        pkg.set_option(name, 0)
        try:
            for _ in range(2):
                assert torch.equal(product(pkg, cuda, A, B, M, N, K, lda=K, ldb=N), want)
        finally:
            pkg.set_option(name, 1)
