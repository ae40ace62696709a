"""The allocation-free entry point ``b200_gemm_f32_static_scratch``.

Some callers cannot call cudaMalloc when they need a product: their loop cannot afford the
implicit synchronisation, or they run under an allocator that was given the whole GPU at start-up.  For them the library
carries its split-K scratch as a fixed array in its own device image.  This test calls that
entry point through the C ABI on shapes that take the split-K path, twice in a row with
different inputs (the second call finds the first call's partial sums still in the scratch),
and checks every result against the ordinary entry point, which gets its workspace from the
caller.  This file sorts last on purpose: a run that stops at the first failure has by then run
every other test."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

STATIC_SCRATCH_BYTES = 4 << 20


def dev(x, cuda):
    import torch

    return torch.from_numpy(np.ascontiguousarray(x)).to(cuda)


def reference_call(pkg, cuda, A, B, M, N, K, **kw):
    import torch

    ws_bytes = pkg.workspace_bytes(1, M, N, K)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=cuda)
    C = torch.full((M, N), float("nan"), device=cuda)
    pkg.gemm(A, B, C, batch=1, M=M, N=N, K=K, ldc=N, workspace=ws, workspace_bytes=ws_bytes, **kw)
    return C, ws_bytes


def test_static_scratch_matches_allocating_entry_point_on_two_calls(pkg, orc, cuda):
    import torch

    g = orc.Rng(77)
    status = torch.zeros(1, dtype=torch.int32, device=cuda)
    # dW = X^T x dY of a 96 -> 384 projection over 2048 tokens, then the conv-style 9 x 50176 x 8
    cases = [dict(M=96, N=384, K=2048, transA=True), dict(M=9, N=8, K=50176, transA=True),
             dict(M=144, N=32, K=12544, transA=False)]
    for round_no in range(2):  # two calls in a row per shape, new inputs each time
        for c in cases:
            M, N, K, tA = c["M"], c["N"], c["K"], c["transA"]
            a = g.randn((K, M) if tA else (M, K))
            b = g.randn((K, N))
            A, B = dev(a, cuda), dev(b, cuda)
            kw = dict(transA=tA, lda=a.shape[1], ldb=N)
            want, ws_bytes = reference_call(pkg, cuda, A, B, M, N, K, **kw)
            assert 0 < ws_bytes <= STATIC_SCRATCH_BYTES, "expected a split-K shape that fits the static scratch"
            got = torch.full((M, N), float("nan"), device=cuda)
            pkg.gemm_static_scratch(A, B, got, batch=1, M=M, N=N, K=K, ldc=N, device_status=status, **kw)
            torch.cuda.synchronize()
            pkg.status()
            assert int(status.item()) == 0, "a device-side wait ran out"
            # same plan, same split, same summation order: identical, and within the parity
            # tolerance of the CPU oracle like every other product
            assert torch.equal(got, want)
            opa = np.ascontiguousarray(a.T) if tA else a
            assert orc.scaled_error(got.cpu().numpy(), orc.matmul(opa, b)) <= orc.parity_tolerance(K)


def test_static_scratch_also_runs_products_that_need_no_scratch(pkg, orc, cuda):
    import torch

    g = orc.Rng(78)
    a, b = g.randn((300, 100)), g.randn((100, 520))
    A, B = dev(a, cuda), dev(b, cuda)
    got = torch.empty((300, 520), device=cuda)
    pkg.gemm_static_scratch(A, B, got, batch=1, M=300, N=520, K=100, lda=100, ldb=520, ldc=520)
    pkg.status()
    assert torch.equal(got, pkg.matmul(A, B))


def test_static_scratch_runs_the_deepest_split_that_fits(pkg, orc, cuda):
    """With ample workspace this shape splits 74 ways (9.7 MB of partial sums); the fixed 4 MiB holds
    32 parts.  The entry point runs that shallower split — the plan b200_gemm_f32 makes when it is
    handed the same 4 MiB — instead of refusing or silently dropping to an unsplit product."""
    import torch

    M, N, K = 128, 256, 16384
    assert pkg.workspace_bytes(1, M, N, K) > STATIC_SCRATCH_BYTES
    plan = pkg.plan(1, M, N, K, STATIC_SCRATCH_BYTES)
    assert plan["split_k"] > 1 and plan["workspace_used"] <= STATIC_SCRATCH_BYTES
    g = orc.Rng(79)
    for _ in range(2):
        a, b = g.randn((M, K), 0.0, K ** -0.5), g.randn((K, N))
        A, B = dev(a, cuda), dev(b, cuda)
        ws = torch.empty(STATIC_SCRATCH_BYTES, dtype=torch.uint8, device=cuda)
        want = torch.full((M, N), float("nan"), device=cuda)
        pkg.gemm(A, B, want, batch=1, M=M, N=N, K=K, lda=K, ldb=N, ldc=N, workspace=ws,
                 workspace_bytes=STATIC_SCRATCH_BYTES)
        got = torch.full((M, N), float("nan"), device=cuda)
        pkg.gemm_static_scratch(A, B, got, batch=1, M=M, N=N, K=K, lda=K, ldb=N, ldc=N)  # no status pointer
        pkg.status()  # also reads the status word inside the library that such calls report to
        assert torch.equal(got, want)
        cpu = orc.matmul(a, b)
        assert orc.scaled_error(got.cpu().numpy(), cpu) <= orc.parity_tolerance(K)
        orc.assert_no_further_from_fp64(got.cpu().numpy(), cpu, a.astype(np.float64) @ b.astype(np.float64))


def test_static_scratch_last_wave_split(pkg, orc, cuda):
    """A product whose mostly empty last wave of tiles is split along K: 1536 x 3328 is 78 tiles of
    256 x 256 on 74 SM pairs, and the four tiles of the second wave run four-way split with exactly
    4 MiB of partial sums — through the fixed scratch, twice."""
    import torch

    M, N, K = 1536, 3328, 1024
    plan = pkg.plan(1, M, N, K, STATIC_SCRATCH_BYTES)
    if not (plan["tail_tiles"] > 0 and 0 < plan["workspace_used"] <= STATIC_SCRATCH_BYTES):
        pytest.skip(f"this GPU's SM count gives another plan: {plan}")
    g = orc.Rng(80)
    for _ in range(2):
        a, b = g.randn((M, K), 0.0, K ** -0.5), g.randn((K, N))
        A, B = dev(a, cuda), dev(b, cuda)
        ws = torch.empty(STATIC_SCRATCH_BYTES, dtype=torch.uint8, device=cuda)
        want = torch.full((M, N), float("nan"), device=cuda)
        pkg.gemm(A, B, want, batch=1, M=M, N=N, K=K, lda=K, ldb=N, ldc=N, workspace=ws,
                 workspace_bytes=STATIC_SCRATCH_BYTES)
        got = torch.full((M, N), float("nan"), device=cuda)
        pkg.gemm_static_scratch(A, B, got, batch=1, M=M, N=N, K=K, lda=K, ldb=N, ldc=N)
        pkg.status()
        assert torch.equal(got, want)
        rows = np.arange(0, M, 37)
        assert orc.scaled_error(got.cpu().numpy()[rows], orc.matmul(a[rows], b)) <= orc.parity_tolerance(K)


def test_static_scratch_refuses_a_forced_split_beyond_its_size(pkg, cuda):
    """Only a split that the caller forced through the "split_k" option and that needs more than
    the fixed 4 MiB is refused (there is no honest way to run it); automatic plans adapt."""
    import torch

    A = torch.zeros((512, 4096), device=cuda)
    B = torch.zeros((4096, 512), device=cuda)
    C = torch.zeros((512, 512), device=cuda)
    pkg.set_option("split_k", 32)
    pkg.set_option("pair_mode", 1)
    try:
        with pytest.raises(pkg.B200Error) as err:
            pkg.gemm_static_scratch(A, B, C, batch=1, M=512, N=512, K=4096, lda=4096, ldb=512, ldc=512)
        assert err.value.code == -3 and "4 MiB" in str(err.value)
    finally:
        pkg.set_option("split_k", 0)
        pkg.set_option("pair_mode", 0)
