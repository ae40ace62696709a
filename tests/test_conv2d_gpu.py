"""Conv2d forward as one implicit-GEMM kernel, against (a) the reference's PyTorch golden vectors
(tests/test_reference.cpp:216-251, abs 1e-4) and (b) the reference's own construction — im2col,
product with the transposed (outC, K) weight view, bias broadcast, (N, spatial, C) -> (N, C, H, W)
permute (src/conv.cpp:280-338) — evaluated with the CPU oracle."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def dev(x, cuda):
    import torch

    return torch.from_numpy(np.ascontiguousarray(x)).to(cuda)


def im2col(x, kh, kw, stride, pad):
    """nn::im2col (src/conv.cpp:61-150): rows (n, oh, ow), columns (c, kh, kw), zeros outside."""
    n, c, h, w = x.shape
    oh, ow = (h + 2 * pad - kh) // stride + 1, (w + 2 * pad - kw) // stride + 1
    xp = np.pad(x, ((0, 0), (0, 0), (pad, pad), (pad, pad)))
    cols = np.empty((n, oh, ow, c, kh, kw), np.float32)
    for i in range(kh):
        for j in range(kw):
            cols[:, :, :, :, i, j] = xp[:, :, i:i + stride * oh:stride, j:j + stride * ow:stride].transpose(0, 2, 3, 1)
    return cols.reshape(n * oh * ow, c * kh * kw), oh, ow


def reference_conv(orc, x, w, b, stride, pad, relu=False):
    out_c, c, kh, kw = w.shape
    cols, oh, ow = im2col(x, kh, kw, stride, pad)
    out = orc.matmul(cols, np.ascontiguousarray(w.reshape(out_c, -1).T))
    if b is not None:
        out = out + b
    if relu:
        out = np.maximum(out, np.float32(0))
    n = x.shape[0]
    return np.ascontiguousarray(out.reshape(n, oh * ow, out_c).transpose(0, 2, 1)).reshape(n, out_c, oh, ow)


def test_pytorch_golden_conv2d(pkg, cuda, golden_dir):
    z = np.load(golden_dir / "pytorch_conv2d.npz")
    for name, stride, pad in [("conv2d_pad1", 1, 1), ("conv2d_stride2", 2, 0)]:
        y = pkg.conv2d(dev(z[f"{name}/input"], cuda), dev(z[f"{name}/weight"], cuda), dev(z[f"{name}/bias"], cuda),
                       stride=stride, padding=pad)
        pkg.status()
        assert y.shape == z[f"{name}/output"].shape
        assert np.max(np.abs(y.cpu().numpy() - z[f"{name}/output"])) <= 1e-4


@pytest.mark.parametrize("shape", [
    # (n, c, h, w, out_c, k, stride, pad)
    (64, 1, 28, 28, 8, 3, 1, 1),     # MNIST-style conv1: K = 9
    (64, 8, 14, 14, 16, 3, 1, 1),    # conv2: K = 72
    (64, 1, 28, 28, 16, 3, 1, 1),    # mnist_demo widths
    (3, 5, 17, 13, 7, 3, 2, 0),      # odd everything, stride 2
    (2, 3, 9, 9, 40, 5, 1, 2),       # 5x5 window, more channels than a 32-wide tile
    (1, 130, 6, 6, 70, 1, 1, 0),     # 1x1 convolution, K > 128
    (1, 520, 5, 5, 12, 3, 1, 1),     # K = 4680: past the per-CTA gather tables, the division path
])
@pytest.mark.parametrize("relu", [False, True])
def test_against_reference_construction(pkg, orc, cuda, shape, relu):
    n, c, h, w, out_c, k, stride, pad = shape
    g = orc.Rng(50)
    x = g.rand((n, c, h, w), 0.0, 1.0)
    bound = float(np.sqrt(6.0 / (c * k * k)))
    wt = g.rand((out_c, c, k, k), -bound, bound)
    b = g.randn((out_c,))
    want = reference_conv(orc, x, wt, b, stride, pad, relu)
    before = pkg.launch_count()
    y = pkg.conv2d(dev(x, cuda), dev(wt, cuda), dev(b, cuda), stride=stride, padding=pad, relu=relu)
    pkg.status()
    assert pkg.launch_count() == before + 1, "the whole layer is one kernel"
    assert orc.scaled_error(y.cpu().numpy(), want) <= orc.parity_tolerance(c * k * k)


def test_exact_on_integers_and_no_bias(pkg, orc, cuda):
    rng = np.random.default_rng(4)
    x = rng.integers(-4, 5, size=(5, 3, 11, 10)).astype(np.float32)
    w = rng.integers(-3, 4, size=(6, 3, 3, 3)).astype(np.float32)
    want = reference_conv(orc, x, w, None, 1, 1)
    y = pkg.conv2d(dev(x, cuda), dev(w, cuda), None, stride=1, padding=1)
    pkg.status()
    assert np.array_equal(y.cpu().numpy(), want)


def test_argument_errors_mirror_the_layer(pkg, cuda):
    import torch

    x = torch.zeros((2, 3, 8, 8), device=cuda)
    with pytest.raises(ValueError):
        pkg.conv2d(x[0], torch.zeros((4, 3, 3, 3), device=cuda))          # not 4-D
    with pytest.raises(ValueError):
        pkg.conv2d(x, torch.zeros((4, 2, 3, 3), device=cuda))             # channel mismatch
    with pytest.raises(ValueError):
        pkg.conv2d(x, torch.zeros((4, 3, 3, 3), device=cuda), stride=0)
