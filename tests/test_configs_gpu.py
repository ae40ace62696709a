"""GPU parity on the benchmark configurations: the char-LM GEMM set, the CNN im2col GEMMs,
the relu-sparse 2048^3 products in all three forms, and size-independent properties at the
full 4096^3 size."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def dev(x, cuda):
    import torch

    return torch.from_numpy(np.ascontiguousarray(x)).to(cuda)


def check(pkg, orc, cuda, a, b, K, backward=True):
    got = pkg.matmul(dev(a, cuda), dev(b, cuda))
    pkg.status()
    want = orc.matmul(a, b)
    got = got.cpu().numpy()
    assert orc.scaled_error(got, want) <= orc.parity_tolerance(K)
    a64, b64 = a.astype(np.float64), b.astype(np.float64)
    orc.assert_no_further_from_fp64(got, want, np.matmul(a64, b64))
    if backward:
        g = orc.Rng(99).randn(want.shape)
        dA, dB = pkg.matmul_backward(dev(a, cuda), dev(b, cuda), dev(g, cuda))
        pkg.status()
        wa, wb = orc.matmul_backward(a, b, g)
        kb = max(want.shape[-1], int(np.prod(want.shape[:-1])))
        dA, dB = dA.cpu().numpy(), dB.cpu().numpy()
        assert orc.scaled_error(dA, wa) <= orc.parity_tolerance(want.shape[-1])
        assert orc.scaled_error(dB, wb) <= orc.parity_tolerance(kb)
        g64 = g.astype(np.float64)
        orc.assert_no_further_from_fp64(dA, wa, np.matmul(g64, np.swapaxes(b64, -1, -2)))
        if b.ndim == 2 and a.ndim > 2:  # shared weight: its gradient sums over the batch (fold_leading)
            ref_b = np.matmul(np.swapaxes(a64, -1, -2), g64).sum(axis=tuple(range(a.ndim - 2)))
            orc.assert_no_further_from_fp64(dB, wb, ref_b)
        elif a.ndim == b.ndim:
            orc.assert_no_further_from_fp64(dB, wb, np.matmul(np.swapaxes(a64, -1, -2), g64))


def xavier(g, fan_in, fan_out):
    bound = float(np.sqrt(6.0 / (fan_in + fan_out)))
    return g.rand((fan_in, fan_out), -bound, bound)


def test_charlm_projection_set(pkg, orc, cuda):
    """batch 32, context 64, d_model 96, FFN 384 (and the reference demo's 192), vocab 121:
    forward, dX (NT) and dW (TN, tall-skinny) for every projection."""
    g = orc.Rng(2)
    x = g.randn((2048, 96))
    for n in (96, 288, 384, 192, 121):
        check(pkg, orc, cuda, x, xavier(g, 96, n), 96)
    for k in (384, 192):
        h = np.maximum(g.randn((2048, k)), 0.0).astype(np.float32)  # post-ReLU: ~50 % exact zeros
        check(pkg, orc, cuda, h, xavier(g, k, 96), k)
    # Linear on a (B, S, d) activation: the weight is shared across the batch
    check(pkg, orc, cuda, g.randn((32, 64, 96)), xavier(g, 96, 121), 96)


def test_charlm_attention_set(pkg, orc, cuda):
    """Per-head batched products, 32 x 4 heads of (64 x 24): Q.K^T and P.V with their four
    backward products."""
    g = orc.Rng(2)
    q, k, v = g.randn((128, 64, 24)), g.randn((128, 64, 24)), g.randn((128, 64, 24))
    kt = np.ascontiguousarray(k.transpose(0, 2, 1))
    check(pkg, orc, cuda, q, kt, 24)
    s = g.randn((128, 64, 64))
    p = np.exp(s - s.max(-1, keepdims=True))
    p = (p / p.sum(-1, keepdims=True)).astype(np.float32)
    check(pkg, orc, cuda, p, v, 64)
    # Q.K^T as one NT call on K as stored, no materialised transpose
    import torch

    scores = torch.empty((128, 64, 64), device=cuda)
    pkg.gemm(dev(q, cuda), dev(k, cuda), scores, batch=128, M=64, N=64, K=24, transB=True, lda=24, ldb=24,
             ldc=64, strideA=64 * 24, strideB=64 * 24, strideC=64 * 64)
    pkg.status()
    assert orc.scaled_error(scores.cpu().numpy(), orc.matmul(q, kt)) <= 1e-5


def test_cnn_im2col_set(pkg, orc, cuda):
    """batch 64 of 28x28: conv1 (50176 x 9 x 8), conv2 (12544 x 72 x 16), dense 784 -> 10, with
    the dW (TN, long contraction) and dX (NT) products.  Column matrices have the zero borders
    of padding 1."""
    g = orc.Rng(3)

    def im2col(x, k=3, pad=1):
        n, c, h, w = x.shape
        xp = np.pad(x, ((0, 0), (0, 0), (pad, pad), (pad, pad)))
        cols = np.empty((n, h, w, c, k, k), np.float32)
        for i in range(k):
            for j in range(k):
                cols[:, :, :, :, i, j] = xp[:, :, i:i + h, j:j + w].transpose(0, 2, 3, 1)
        return cols.reshape(n * h * w, c * k * k)

    def he(g, out_c, fan_in):
        bound = float(np.sqrt(6.0 / fan_in))
        return g.rand((out_c, fan_in), -bound, bound)

    x1 = g.rand((64, 1, 28, 28), 0.0, 1.0)
    w1 = he(g, 8, 9)
    cols1 = im2col(x1)
    check(pkg, orc, cuda, cols1, np.ascontiguousarray(w1.T), 9)
    x2 = g.rand((64, 8, 14, 14), 0.0, 1.0)
    w2 = he(g, 16, 72)
    check(pkg, orc, cuda, im2col(x2), np.ascontiguousarray(w2.T), 72)
    check(pkg, orc, cuda, g.rand((64, 784), 0.0, 1.0), xavier(g, 784, 10), 784)
    # cols x W^T with W as stored (outC x K): the NT form Conv2d::forward needs
    import torch

    out = torch.empty((cols1.shape[0], 8), device=cuda)
    pkg.gemm(dev(cols1, cuda), dev(w1, cuda), out, batch=1, M=cols1.shape[0], N=8, K=9, transB=True, lda=9,
             ldb=9, ldc=8)
    pkg.status()
    assert orc.scaled_error(out.cpu().numpy(), orc.matmul(cols1, np.ascontiguousarray(w1.T))) <= 1e-5


@pytest.mark.parametrize("form", ["NN", "NT", "TN"])
def test_relu_sparse_2048(pkg, orc, cuda, form):
    """A = relu(N(0,1)) (half exact zeros), B dense, seed 4; the reference computes the
    transposed forms by materialising the transpose first."""
    import torch

    g = orc.Rng(4)
    n = 2048
    a = np.maximum(g.randn((n, n)), 0.0).astype(np.float32)
    b = g.randn((n, n))
    tA, tB = form[0] == "T", form[1] == "T"
    opa = np.ascontiguousarray(a.T) if tA else a
    opb = np.ascontiguousarray(b.T) if tB else b
    want = orc.matmul(opa, opb)
    C = torch.empty((n, n), device=cuda)
    pkg.gemm(dev(a, cuda), dev(b, cuda), C, batch=1, M=n, N=n, K=n, transA=tA, transB=tB, lda=n, ldb=n, ldc=n)
    pkg.status()
    got = C.cpu().numpy()
    assert orc.scaled_error(got, want) <= orc.parity_tolerance(n)
    # Against fp64 the kernel is far closer than the reference's own fp32 loop (measured 2.6e-5
    # against 9.7e-5 with a promotion to fp32 registers after every k-block; promoting every 4th
    # k-block gives 6.3e-5): holding it to half the loop's error is what catches a regression of
    # the accumulation scheme, which the wide bound above would let through.
    rows = np.arange(0, n, 16)
    ref64 = (opa[rows].astype(np.float64) @ opb.astype(np.float64))
    err_gpu, err_cpu = orc.scaled_error(got[rows], ref64), orc.scaled_error(want[rows], ref64)
    assert err_gpu <= 0.5 * err_cpu, (err_gpu, err_cpu)


def test_large_square_properties_4096(pkg, orc, cuda):
    """4096^3 on the bytes the reference's own generator produces for this configuration
    (manual_seed(1), then A and B = Tensor::randn({n, n}, 0, 1/sqrt(n)) in that order): sampled rows
    against the CPU oracle at the flat 1e-5 (rows are independent in the reference loop, so those
    rows are exactly what the full product holds) and against fp64, run-to-run bit-identity, and
    linearity in alpha."""
    import torch

    n = 4096
    g = orc.Rng(1)
    a = g.randn((n, n), 0.0, n ** -0.5)
    b = g.randn((n, n), 0.0, n ** -0.5)
    A, B = dev(a, cuda), dev(b, cuda)
    ws_bytes = pkg.workspace_bytes(1, n, n, n)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=cuda)
    C = torch.empty((n, n), device=cuda)
    pkg.gemm(A, B, C, batch=1, M=n, N=n, K=n, lda=n, ldb=n, ldc=n, workspace=ws, workspace_bytes=ws_bytes)
    C2 = torch.empty((n, n), device=cuda)
    pkg.gemm(A, B, C2, batch=1, M=n, N=n, K=n, lda=n, ldb=n, ldc=n, workspace=ws, workspace_bytes=ws_bytes)
    pkg.status()
    assert torch.equal(C, C2)
    rows = np.arange(5, n, 97)
    got = C.cpu().numpy()[rows]
    want = orc.matmul(a[rows], b)
    assert orc.scaled_error(got, want) <= 1e-5
    ref64 = a[rows].astype(np.float64) @ b.astype(np.float64)
    err_gpu, err_cpu = orc.scaled_error(got, ref64), orc.scaled_error(want, ref64)
    assert err_gpu <= 2e-7 and err_gpu <= err_cpu, (err_gpu, err_cpu)
    pkg.gemm(A, B, C2, batch=1, M=n, N=n, K=n, lda=n, ldb=n, ldc=n, alpha=2.0, workspace=ws,
             workspace_bytes=ws_bytes)
    pkg.status()
    assert torch.equal(C2, 2.0 * C)


def test_largest_config_16384(pkg, orc, cuda):
    """Configuration 5 at its full size, 16384^3 with N(0, 1/K) inputs drawn by the reference's generator (3 GiB on the device): sampled rows
    against the CPU loop (rows are independent there, so these are the rows of the full product) and against
    fp64, run-to-run bit-identity, and the plan with the K-split last wave against the plan without it."""
    import torch

    n = 16384
    g = orc.Rng(1)  # the reference generator's bytes: manual_seed(1), then A, then B
    A = dev(g.randn((n, n), 0.0, n ** -0.5), cuda)
    B = dev(g.randn((n, n), 0.0, n ** -0.5), cuda)
    C = torch.empty((n, n), device=cuda)
    pkg.gemm(A, B, C, batch=1, M=n, N=n, K=n, lda=n, ldb=n, ldc=n)
    pkg.status()
    rows = torch.arange(7, n, 683, device=cuda)  # 24 rows
    got = C[rows].cpu().numpy()
    b_host = B.cpu().numpy()
    want = orc.matmul(A[rows].cpu().numpy(), b_host)
    # N(0, 1/K) inputs keep the outputs of order one and the CPU loop's drift small: the flat 1e-5
    # of the reference's parity tests holds at K = 16384 too (measured 3e-7)
    assert orc.scaled_error(got, want) <= 1e-5
    ref64 = (A[rows].double() @ B.double()).cpu().numpy()
    err_gpu, err_cpu = orc.scaled_error(got, ref64), orc.scaled_error(want, ref64)
    assert err_gpu <= 1e-6 and err_gpu <= err_cpu, (err_gpu, err_cpu)
    del b_host, want, ref64
    first = C[rows].clone()
    C.zero_()
    pkg.gemm(A, B, C, batch=1, M=n, N=n, K=n, lda=n, ldb=n, ldc=n)
    pkg.status()
    assert torch.equal(C[rows], first)
    ws_bytes = pkg.workspace_bytes(1, n, n, n)
    if ws_bytes:
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=cuda)
        keep = C[::509].clone()
        C.zero_()
        pkg.gemm(A, B, C, batch=1, M=n, N=n, K=n, lda=n, ldb=n, ldc=n, workspace=ws, workspace_bytes=ws_bytes)
        pkg.status()
        assert orc.scaled_error(C[::509].cpu().numpy(), keep.cpu().numpy()) <= 1e-5
