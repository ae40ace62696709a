"""Stream ordering, concurrent streams, big batch counts and strided batches through the C ABI."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def dev(x, cuda):
    import torch

    return torch.from_numpy(np.ascontiguousarray(x)).to(cuda)


def test_calls_are_ordered_on_the_given_stream(pkg, orc, cuda):
    """A chain y = (x W1) W2 issued on a side stream with no host synchronisation in between."""
    import torch

    g = orc.Rng(60)
    # weights scaled like a layer's (variance 1/fan_in) so that activations stay of order one
    x, w1, w2 = g.randn((300, 200)), g.randn((200, 260), 0.0, 200 ** -0.5), g.randn((260, 90), 0.0, 260 ** -0.5)
    X, W1, W2 = dev(x, cuda), dev(w1, cuda), dev(w2, cuda)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    H = torch.empty((300, 260), device=cuda)
    Y = torch.empty((300, 90), device=cuda)
    with torch.cuda.stream(side):
        pkg.gemm(X, W1, H, batch=1, M=300, N=260, K=200, lda=200, ldb=260, ldc=260, stream=side)
        pkg.gemm(H, W2, Y, batch=1, M=300, N=90, K=260, lda=260, ldb=90, ldc=90, stream=side)
    side.synchronize()
    pkg.status()
    want = orc.matmul(orc.matmul(x, w1), w2)
    assert orc.scaled_error(Y.cpu().numpy(), want) <= orc.parity_tolerance(260)


def test_two_streams_at_once_do_not_interfere(pkg, orc, cuda):
    import torch

    g = orc.Rng(61)
    cases = []
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    for i, (M, K, N) in enumerate([(700, 300, 500), (513, 129, 257)]):
        a, b = g.randn((M, K)), g.randn((K, N))
        A, B = dev(a, cuda), dev(b, cuda)
        C = torch.empty((M, N), device=cuda)
        cases.append((a, b, A, B, C, M, K, N))
    torch.cuda.synchronize()
    for _ in range(3):
        for s, (a, b, A, B, C, M, K, N) in zip(streams, cases):
            pkg.gemm(A, B, C, batch=1, M=M, N=N, K=K, lda=K, ldb=N, ldc=N, stream=s)
    torch.cuda.synchronize()
    pkg.status()
    for a, b, A, B, C, M, K, N in cases:
        assert orc.scaled_error(C.cpu().numpy(), orc.matmul(a, b)) <= orc.parity_tolerance(K)


def test_batch_count_beyond_65535(pkg, orc, cuda):
    """The reference caps the batch at 65535 (grid.z, src/cuda/kernels_common.cuh:59-62); the
    persistent tile walk here does not."""
    import torch

    batch = 70000
    rng = np.random.default_rng(8)
    a = rng.integers(-3, 4, size=(batch, 4, 8)).astype(np.float32)
    b = rng.integers(-3, 4, size=(8, 5)).astype(np.float32)
    got = pkg.matmul(dev(a, cuda), dev(b, cuda))
    pkg.status()
    assert np.array_equal(got.cpu().numpy(), orc.matmul(a, b))


def test_strided_batches_and_views_into_larger_buffers(pkg, orc, cuda):
    """Batch strides larger than a matrix (every second matrix of a buffer) and leading dimensions
    larger than a row: sub-blocks of bigger arrays, no copies."""
    import torch

    g = orc.Rng(62)
    big_a = g.randn((6, 40, 64))   # use batches 0, 2, 4 and columns 8..39 of each
    big_b = g.randn((6, 48, 72))   # rows 0..31, columns 4..67
    A, B = dev(big_a, cuda), dev(big_b, cuda)
    M, K, N, batch = 40, 32, 64, 3
    C = torch.full((batch, M, N), float("nan"), device=cuda)
    a_ptr = A.data_ptr() + 8 * 4
    b_ptr = B.data_ptr() + 4 * 4
    pkg.gemm(a_ptr, b_ptr, C, batch=batch, M=M, N=N, K=K, lda=64, ldb=72, ldc=N, strideA=2 * 40 * 64,
             strideB=2 * 48 * 72, strideC=M * N)
    pkg.status()
    want = orc.matmul(np.ascontiguousarray(big_a[0::2, :, 8:40]), np.ascontiguousarray(big_b[0::2, :32, 4:68]))
    assert orc.scaled_error(C.cpu().numpy(), want) <= 1e-5


def test_nan_and_zero_inputs_propagate_like_arithmetic(pkg, cuda):
    import torch

    A = torch.zeros((130, 70), device=cuda)
    B = torch.ones((70, 50), device=cuda)
    out = pkg.matmul(A, B)
    pkg.status()
    assert not out.cpu().numpy().any()
    A[3, 5] = float("nan")
    out = pkg.matmul(A, B).cpu().numpy()
    assert np.isnan(out[3]).all() and not np.isnan(np.delete(out, 3, axis=0)).any()


def _block_weights(orc, cuda):
    g = orc.Rng(62)
    d, ff = 96, 384
    w = {
        "qkv": g.rand((d, 3 * d), -0.125, 0.125), "bqkv": g.randn((3 * d,), 0.0, 0.1),
        "out": g.rand((d, d), -0.17, 0.17), "bout": g.randn((d,), 0.0, 0.1),
        "ff1": g.rand((d, ff), -0.11, 0.11), "b1": g.randn((ff,), 0.0, 0.1),
        "ff2": g.rand((ff, d), -0.11, 0.11), "b2": g.randn((d,), 0.0, 0.1),
    }
    return {k: dev(v, cuda) for k, v in w.items()}


def _block_products(pkg, x, w, mask):
    """The products of one char-LM Transformer block (B = 32, S = 64, d = 96, 4 heads, FFN 384) as five
    layer calls: fused Q|K|V projection, attention core on its column slices, output projection, FF1 + ReLU, FF2."""
    qkv = pkg.linear(x, w["qkv"], w["bqkv"]).view(32, 64, 288)
    ctx = pkg.multi_head_attention_core(qkv[:, :, :96], qkv[:, :, 96:192], qkv[:, :, 192:], 4, mask)
    o = pkg.linear(ctx.view(2048, 96), w["out"], w["bout"])
    h = pkg.linear(o, w["ff1"], w["b1"], relu=True)
    return pkg.linear(h, w["ff2"], w["b2"])


def test_block_chain_replays_from_a_cuda_graph(pkg, orc, cuda):
    """The launches allocate nothing and synchronise nothing, so a chain of them can be captured once
    and replayed: the replay on new inputs gives, bit for bit, what the eager calls give."""
    import torch

    w = _block_weights(orc, cuda)
    mask = torch.triu(torch.full((64, 64), -1e9, device=cuda), 1)
    g = orc.Rng(63)
    x_static = dev(g.randn((2048, 96)), cuda)
    _block_products(pkg, x_static, w, mask)  # warm-up: per-device set-up happens outside the capture
    pkg.status()
    torch.cuda.synchronize()
    before = pkg.launch_count()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        y_static = _block_products(pkg, x_static, w, mask)
    launches = pkg.launch_count() - before
    assert 5 <= launches <= 7, "one kernel per layer call (plus a reduction where the planner splits K)"
    for seed in (64, 65):
        x_new = dev(orc.Rng(seed).randn((2048, 96)), cuda)
        x_static.copy_(x_new)
        graph.replay()
        torch.cuda.synchronize()
        pkg.status()
        want = _block_products(pkg, x_new, w, mask)
        pkg.status()
        assert torch.equal(y_static, want)
    # and against the reference's sequence of separate steps, evaluated with the CPU oracle
    xn = x_new.cpu().numpy()
    wn = {k: v.cpu().numpy() for k, v in w.items()}
    qkv = (orc.matmul(xn, wn["qkv"]) + wn["bqkv"]).reshape(32, 64, 3, 4, 24).transpose(2, 0, 3, 1, 4)
    scores = orc.matmul(np.ascontiguousarray(qkv[0]), np.ascontiguousarray(qkv[1].transpose(0, 1, 3, 2)))
    scores = scores * np.float32(24 ** -0.5) + mask.cpu().numpy()
    e = np.exp(scores - scores.max(-1, keepdims=True), dtype=np.float32)
    p = (e / e.sum(-1, keepdims=True, dtype=np.float32)).astype(np.float32)
    ctx = orc.matmul(p, np.ascontiguousarray(qkv[2])).transpose(0, 2, 1, 3).reshape(2048, 96)
    o = orc.matmul(np.ascontiguousarray(ctx), wn["out"]) + wn["bout"]
    h = np.maximum(orc.matmul(o, wn["ff1"]) + wn["b1"], np.float32(0))
    ref = orc.matmul(h, wn["ff2"]) + wn["b2"]
    assert orc.scaled_error(y_static.cpu().numpy(), ref) <= 5e-5  # five layers deep
