"""The host-side mirror of Tensor::matmul and its autograd node, on the GPU, against the
reference's PyTorch golden vectors (tests/test_reference.cpp:99-114) and the CPU oracle's
backward (src/tensor_ops.cpp:570-585)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def dev(x, cuda):
    import torch

    return torch.from_numpy(np.ascontiguousarray(x)).to(cuda)


def test_golden_forward_and_gradients(pkg, cuda, golden_dir):
    z = np.load(golden_dir / "pytorch_matmul.npz")
    for name in ["matmul", "matmul_batched", "matmul_shared"]:
        a = pkg.Tensor(dev(z[f"{name}/a"], cuda), requires_grad=True)
        b = pkg.Tensor(dev(z[f"{name}/b"], cuda), requires_grad=True)
        out = a.matmul(b)
        out.backward(dev(z[f"{name}/grad_output"], cuda))
        pkg.status()
        assert np.max(np.abs(out.data.cpu().numpy() - z[f"{name}/output"])) <= 1e-4
        assert np.max(np.abs(a.grad.data.cpu().numpy() - z[f"{name}/grad.a"])) <= 1e-4
        assert np.max(np.abs(b.grad.data.cpu().numpy() - z[f"{name}/grad.b"])) <= 1e-4


@pytest.mark.parametrize("sa,sb", [((33, 65), (65, 17)), ((4, 3, 17, 23), (4, 3, 23, 11)),
                                   ((8, 12, 40), (40, 20)), ((40, 12), (5, 12, 7))])
def test_backward_forms_against_oracle(pkg, orc, cuda, sa, sb):
    g = orc.Rng(21)
    a, b = g.randn(sa), g.randn(sb)
    want = orc.matmul(a, b)
    go = g.randn(want.shape)
    wa, wb = orc.matmul_backward(a, b, go)
    dA, dB = pkg.matmul_backward(dev(a, cuda), dev(b, cuda), dev(go, cuda))
    pkg.status()
    assert dA.shape == tuple(sa) and dB.shape == tuple(sb)
    assert orc.scaled_error(dA.cpu().numpy(), wa) <= 1e-5
    assert orc.scaled_error(dB.cpu().numpy(), wb) <= 1e-5


def test_chain_of_products_accumulates_gradients(pkg, orc, cuda):
    """y = (x W1) W2 with x used twice: gradients add up (first write copies, later add)."""
    g = orc.Rng(22)
    x, w1, w2 = g.randn((16, 24)), g.randn((24, 24)), g.randn((24, 8))
    X = pkg.Tensor(dev(x, cuda), requires_grad=True)
    W1 = pkg.Tensor(dev(w1, cuda), requires_grad=True)
    W2 = pkg.Tensor(dev(w2, cuda), requires_grad=True)
    y = X.matmul(W1).matmul(W2)
    go = g.randn((16, 8))
    y.backward(dev(go, cuda))
    pkg.status()
    h = orc.matmul(x, w1)
    dh, dw2 = orc.matmul_backward(h, w2, go)
    dx, dw1 = orc.matmul_backward(x, w1, dh)
    assert orc.scaled_error(W2.grad.data.cpu().numpy(), dw2) <= 1e-5
    assert orc.scaled_error(W1.grad.data.cpu().numpy(), dw1) <= 1e-4
    assert orc.scaled_error(X.grad.data.cpu().numpy(), dx) <= 1e-4


def test_fused_multi_destination_stores(pkg, orc, cuda):
    """The column-shard entry point writes the same tiles to every destination buffer (on one
    GPU the 'peers' are just further local buffers)."""
    import torch

    g = orc.Rng(23)
    M, K, N = 200, 64, 256
    a, b = g.randn((M, K)), g.randn((K, N))
    A, B = dev(a, cuda), dev(b, cuda)
    dests = [torch.full((M, N), float("nan"), device=cuda) for _ in range(3)]
    for rank in range(2):
        col0, cols = pkg.shard.column_shard(N, 2, rank)
        pkg.gemm_colshard(A, B, dests, M=M, N=N, K=K, col0=col0, cols=cols, lda=K, ldb=N, ldc=N)
    pkg.status()
    want = orc.matmul(a, b)
    for d in dests:
        assert orc.scaled_error(d.cpu().numpy(), want) <= 1e-5
    assert torch.equal(dests[0], dests[1]) and torch.equal(dests[1], dests[2])
    # the sharded result is bit-identical to the unsharded product
    whole = pkg.matmul(A, B)
    pkg.status()
    assert torch.equal(whole, dests[0])


@pytest.mark.parametrize("M,N,K", [(12288, 4096, 256), (25600, 768, 100), (1000, 1056, 72)])
def test_eight_destinations_several_tiles_per_cta(pkg, cuda, M, N, K):
    """Eight shards into eight destination buffers, the widest gather the library accepts, on shapes
    whose shards give a CTA more than one tile (CTA pairs; single CTAs; a ragged small one), so that
    the forwarder warps follow the workers across tiles: every buffer ends bit-identical to the
    unsharded product."""
    import torch

    gen = torch.Generator(device="cpu").manual_seed(M + N + K)
    A = torch.randn((M, K), generator=gen).to(cuda)
    B = torch.randn((K, N), generator=gen).to(cuda)
    dests = [torch.full((M, N), float("nan"), device=cuda) for _ in range(8)]
    for rank in range(8):
        col0, cols = pkg.shard.column_shard(N, 8, rank)
        # each "rank" lists its own buffer first, as the sharded call does
        order = dests[rank:] + dests[:rank]
        pkg.gemm_colshard(A, B, order, M=M, N=N, K=K, col0=col0, cols=cols, lda=K, ldb=N, ldc=N)
    pkg.status()
    whole = pkg.matmul(A, B)
    pkg.status()
    for d in dests:
        assert torch.equal(d, whole)
