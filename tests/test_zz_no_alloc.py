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


def test_static_scratch_refuses_plans_beyond_its_size(pkg, cuda):
    import torch

    A = torch.zeros((512, 4096), device=cuda)
    B = torch.zeros((4096, 512), device=cuda)
    C = torch.zeros((512, 512), device=cuda)
    pkg.set_option("split_k", 32)
    pkg.set_option("pair_mode", 1)
    try:
        assert pkg.workspace_bytes(1, 512, 512, 4096) > STATIC_SCRATCH_BYTES
        with pytest.raises(pkg.B200Error) as err:
            pkg.gemm_static_scratch(A, B, C, batch=1, M=512, N=512, K=4096, lda=4096, ldb=512, ldc=512)
        assert err.value.code == -3 and "4 MiB" in str(err.value)
    finally:
        pkg.set_option("split_k", 0)
        pkg.set_option("pair_mode", 0)
