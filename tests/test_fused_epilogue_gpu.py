"""The fused epilogue (bias, scale + additive mask, ReLU) against the reference's sequence of
separate operations: the CPU oracle's product followed by the same fp32 element-wise steps in the
same order (src/nn.cpp:119-122, src/transformer.cpp:292-297, :413)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def dev(x, cuda):
    import torch

    return torch.from_numpy(np.ascontiguousarray(x)).to(cuda)


@pytest.mark.parametrize("rows,k,n", [(2048, 96, 384), (2048, 96, 121), (64, 784, 10), (300, 100, 520)])
@pytest.mark.parametrize("relu", [False, True])
def test_linear_bias_relu(pkg, orc, cuda, rows, k, n, relu):
    g = orc.Rng(40)
    x, w, b = g.randn((rows, k)), g.randn((k, n)), g.randn((n,))
    want = orc.matmul(x, w) + b  # fp32 add of the broadcast bias, as Linear::forward does
    if relu:
        want = np.maximum(want, np.float32(0.0))
    got = pkg.linear(dev(x, cuda), dev(w, cuda), dev(b, cuda), relu=relu)
    pkg.status()
    assert orc.scaled_error(got.cpu().numpy(), want) <= orc.parity_tolerance(k)
    if relu:
        assert (got >= 0).all()


def test_linear_3d_input_and_integer_exactness(pkg, orc, cuda):
    rng = np.random.default_rng(3)
    x = rng.integers(-4, 5, size=(4, 33, 40)).astype(np.float32)
    w = rng.integers(-3, 4, size=(40, 24)).astype(np.float32)
    b = rng.integers(-9, 10, size=(24,)).astype(np.float32)
    want = np.maximum(orc.matmul(x.reshape(-1, 40), w) + b, 0).reshape(4, 33, 24)
    got = pkg.linear(dev(x, cuda), dev(w, cuda), dev(b, cuda), relu=True)
    pkg.status()
    assert np.array_equal(got.cpu().numpy(), want)


@pytest.mark.parametrize("causal", [False, True])
def test_attention_scores_scale_and_mask(pkg, orc, cuda, causal):
    g = orc.Rng(41)
    q, k = g.randn((32, 4, 64, 24)), g.randn((32, 4, 64, 24))
    scale = np.float32(1.0 / np.sqrt(24.0))
    mask = np.triu(np.full((64, 64), -1e9, np.float32), 1) if causal else None
    want = orc.matmul(q.reshape(128, 64, 24), np.ascontiguousarray(k.reshape(128, 64, 24).transpose(0, 2, 1)))
    want = want * scale  # Tensor * scalar, then + mask: two fp32 operations
    if causal:
        want = want + mask
    got = pkg.attention_scores(dev(q, cuda), dev(k, cuda), float(scale), dev(mask, cuda) if causal else None)
    pkg.status()
    got = got.cpu().numpy().reshape(128, 64, 64)
    assert orc.scaled_error(got, want) <= 1e-5
    if causal:
        assert (got[:, np.triu_indices(64, 1)[0], np.triu_indices(64, 1)[1]] < -1e8).all()


def test_fused_epilogue_on_split_k_and_tail_paths(pkg, orc, cuda):
    """The reductions of the split-K and tail-wave plans apply the same epilogue."""
    import torch

    g = orc.Rng(42)
    for (M, N, K) in [(96, 384, 2048), (2560, 2048, 1024)]:
        a, b, bias = g.randn((M, K)), g.randn((K, N)), g.randn((N,))
        add = g.randn((M, N))
        ws_bytes = pkg.workspace_bytes(1, M, N, K)
        assert ws_bytes > 0
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=cuda)
        C = torch.empty((M, N), device=cuda)
        pkg.gemm_fused(dev(a, cuda), dev(b, cuda), C, batch=1, M=M, N=N, K=K, lda=K, ldb=N, ldc=N, alpha=0.5,
                       bias=dev(bias, cuda), addend=dev(add, cuda), ld_addend=N, relu=True, workspace=ws,
                       workspace_bytes=ws_bytes)
        pkg.status()
        want = np.maximum((orc.matmul(a, b) * np.float32(0.5) + bias) + add, 0)
        assert orc.scaled_error(C.cpu().numpy(), want) <= orc.parity_tolerance(K)


def test_epilogue_argument_errors(pkg, cuda):
    import torch

    A = torch.zeros((8, 8), device=cuda)
    with pytest.raises(pkg.B200Error):
        pkg.gemm_fused(A, A, torch.empty((8, 8), device=cuda), batch=1, M=8, N=8, K=8, lda=8, ldb=8, ldc=8,
                       addend=A, ld_addend=4)
    with pytest.raises(ValueError):
        pkg.linear(A, A, torch.zeros(3, device=cuda))
