"""Conv2d's gradients as implicit-GEMM kernels — no column matrix, no transposes, no col2im scatter —
against (a) the reference's PyTorch golden vectors (tests/test_reference.cpp:216-251, abs 1e-4),
(b) recorded outputs of the unmodified reference engine's Conv2d + autograd, and (c) the reference's
construction (product backward over im2col's columns, col2im; src/tensor_ops.cpp:570-585,
src/conv.cpp:152-257) evaluated with the CPU oracle on seeded inputs."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def dev(x, cuda):
    import torch

    return torch.from_numpy(np.ascontiguousarray(x)).to(cuda)


def test_pytorch_golden_conv2d_gradients(pkg, cuda, golden_dir):
    z = np.load(golden_dir / "pytorch_conv2d.npz")
    for name, stride, pad in [("conv2d_pad1", 1, 1), ("conv2d_stride2", 2, 0)]:
        gx, gw, gb = pkg.conv2d_backward(dev(z[f"{name}/input"], cuda), dev(z[f"{name}/weight"], cuda),
                                         dev(z[f"{name}/grad_output"], cuda), stride=stride, padding=pad)
        pkg.status()
        assert np.max(np.abs(gx.cpu().numpy() - z[f"{name}/grad.input"])) <= 1e-4
        assert np.max(np.abs(gw.cpu().numpy() - z[f"{name}/grad.weight"])) <= 1e-4
        assert np.max(np.abs(gb.cpu().numpy() - z[f"{name}/grad.bias"])) <= 1e-4


def test_recorded_reference_engine_gradients(pkg, orc, cuda, golden_dir):
    z = np.load(golden_dir / "reference_conv_backward.npz")
    for tag in ("pad1", "stride2", "k5pad2"):
        stride, pad = (int(v) for v in z[f"{tag}/window"])
        x, wt, dy = z[f"{tag}/x"], z[f"{tag}/weight"], z[f"{tag}/grad_output"]
        gx, gw, gb = pkg.conv2d_backward(dev(x, cuda), dev(wt, cuda), dev(dy, cuda), stride=stride, padding=pad)
        pkg.status()
        positions = dy.shape[0] * dy.shape[2] * dy.shape[3]
        assert orc.scaled_error(gx.cpu().numpy(), z[f"{tag}/grad.x"]) <= 1e-5
        assert orc.scaled_error(gw.cpu().numpy(), z[f"{tag}/grad.weight"]) <= orc.parity_tolerance(positions)
        assert orc.scaled_error(gb.cpu().numpy(), z[f"{tag}/grad.bias"]) <= orc.parity_tolerance(positions)


SHAPES = [
    # (n, c, h, w, out_c, k, stride, pad)
    (64, 1, 28, 28, 8, 3, 1, 1),     # MNIST-style conv1: 50176 positions, K = 9
    (64, 8, 14, 14, 16, 3, 1, 1),    # conv2: 12544 positions, K = 72
    (3, 5, 17, 13, 7, 3, 2, 0),      # odd everything, stride 2 (positions not a multiple of 4)
    (2, 3, 9, 9, 40, 5, 1, 2),       # 5x5 window, more channels than a 32-wide tile
    (1, 130, 6, 6, 70, 1, 1, 0),     # 1x1 convolution, more than 128 input channels
    (2, 4, 7, 9, 3, 2, 3, 1),        # stride larger than the window: some pixels get no gradient
    (2, 3, 8, 8, 150, 3, 1, 1),      # more than 128 output channels (two row tiles of the weight gradient)
    (1, 6, 5, 5, 460, 3, 1, 1),      # outC*kH*kW = 4140: the input gradient's gather leaves the tables
    (1, 520, 5, 5, 12, 3, 1, 1),     # C*kH*kW = 4680 columns in the weight gradient
]


@pytest.mark.parametrize("shape", SHAPES)
def test_against_reference_construction(pkg, orc, cuda, shape):
    n, c, h, w, out_c, k, stride, pad = shape
    g = orc.Rng(51)
    x = g.rand((n, c, h, w), 0.0, 1.0)
    bound = float(np.sqrt(6.0 / (c * k * k)))
    wt = g.rand((out_c, c, k, k), -bound, bound)
    oh, ow = (h + 2 * pad - k) // stride + 1, (w + 2 * pad - k) // stride + 1
    dy = g.randn((n, out_c, oh, ow))
    want_x, want_w, want_b = orc.conv2d_backward(x, wt, dy, stride, pad)
    before = pkg.launch_count()
    gx, gw, gb = pkg.conv2d_backward(dev(x, cuda), dev(wt, cuda), dev(dy, cuda), stride=stride, padding=pad)
    pkg.status()
    assert pkg.launch_count() - before <= 3, "weight gradient with the bias column, its reduction, input gradient"
    positions = n * oh * ow
    assert orc.scaled_error(gx.cpu().numpy(), want_x) <= orc.parity_tolerance(out_c * k * k)
    assert orc.scaled_error(gw.cpu().numpy(), want_w) <= orc.parity_tolerance(positions)
    assert orc.scaled_error(gb.cpu().numpy(), want_b) <= orc.parity_tolerance(positions)


def test_exact_on_integers(pkg, orc, cuda):
    """Small integers: every product and partial sum is exact in fp32, so any summation order gives
    the reference's gradients bit for bit."""
    rng = np.random.default_rng(6)
    x = rng.integers(-4, 5, size=(5, 3, 11, 10)).astype(np.float32)
    w = rng.integers(-3, 4, size=(6, 3, 3, 3)).astype(np.float32)
    for stride, pad in ((1, 1), (2, 0), (2, 1)):
        oh, ow = (11 + 2 * pad - 3) // stride + 1, (10 + 2 * pad - 3) // stride + 1
        dy = rng.integers(-3, 4, size=(5, 6, oh, ow)).astype(np.float32)
        want = orc.conv2d_backward(x, w, dy, stride, pad)
        got = pkg.conv2d_backward(dev(x, cuda), dev(w, cuda), dev(dy, cuda), stride=stride, padding=pad)
        pkg.status()
        for a, b in zip(got, want):
            assert np.array_equal(a.cpu().numpy(), b)


def test_accumulates_into_existing_gradients(pkg, orc, cuda):
    """Tensor::add_grad (src/tensor.cpp:168-203): a second backward adds to the stored gradient."""
    n, c, h, w, out_c, k = 4, 3, 12, 12, 5, 3
    g = orc.Rng(52)
    x, wt = g.randn((n, c, h, w)), g.randn((out_c, c, k, k))
    dy1, dy2 = g.randn((n, out_c, h, w)), g.randn((n, out_c, h, w))
    dx, dwt, ddy1, ddy2 = dev(x, cuda), dev(wt, cuda), dev(dy1, cuda), dev(dy2, cuda)
    first = pkg.conv2d_backward(dx, dwt, ddy1, stride=1, padding=1)
    second = pkg.conv2d_backward(dx, dwt, ddy2, stride=1, padding=1)
    acc = tuple(t.clone() for t in first)
    pkg.conv2d_backward(dx, dwt, ddy2, stride=1, padding=1, accumulate_into=acc)
    pkg.status()
    for a, f, s in zip(acc, first, second):
        assert np.max(np.abs(a.cpu().numpy() - (f + s).cpu().numpy())) <= 1e-5 * max(1.0, float(f.abs().max()))


def test_optional_gradients_and_unsplit_weight_gradient(pkg, orc, cuda):
    import torch

    n, c, h, w, out_c, k = 8, 2, 10, 10, 4, 3
    g = orc.Rng(53)
    x, wt, dy = g.randn((n, c, h, w)), g.randn((out_c, c, k, k)), g.randn((n, out_c, h, w))
    want_x, want_w, want_b = orc.conv2d_backward(x, wt, dy, 1, 1)
    gx, gw, gb = pkg.conv2d_backward(dev(x, cuda), dev(wt, cuda), dev(dy, cuda), stride=1, padding=1,
                                     need_input_grad=False, need_bias_grad=False)
    assert gx is None and gb is None
    assert orc.scaled_error(gw.cpu().numpy(), want_w) <= orc.parity_tolerance(n * h * w)
    # straight through the C ABI without a workspace: the weight gradient runs unsplit
    gw2 = torch.empty_like(gw)
    pkg.lib.conv2d_backward(dev(x, cuda), None, dev(dy, cuda), None, gw2, None, n=n, c=c, h=h, w=w, out_c=out_c, kh=k,
                            kw=k, stride=1, pad=1)
    pkg.status()
    assert orc.scaled_error(gw2.cpu().numpy(), want_w) <= orc.parity_tolerance(n * h * w)


def test_argument_errors(pkg, cuda):
    import torch

    x = torch.zeros((2, 3, 8, 8), device=cuda)
    w = torch.zeros((4, 3, 3, 3), device=cuda)
    with pytest.raises(ValueError):
        pkg.conv2d_backward(x, w, torch.zeros((2, 4, 8, 8), device=cuda))                 # no padding: dy is 6 x 6
    with pytest.raises(ValueError):
        pkg.conv2d_backward(x, torch.zeros((4, 2, 3, 3), device=cuda), torch.zeros((2, 4, 6, 6), device=cuda))
    with pytest.raises(ValueError):
        pkg.conv2d_backward(x, w, torch.zeros((2, 4, 6, 6), device=cuda), stride=0)


def test_tf32_mode_is_coarser_but_close(pkg, orc, cuda):
    """The opt-in TF32 mode of the convolution kernels (forward and the three gradients)."""
    n, c, h, w, out_c, k = 8, 8, 14, 14, 16, 3
    g = orc.Rng(54)
    x, wt, b = g.rand((n, c, h, w), 0.0, 1.0), g.rand((out_c, c, k, k), -0.3, 0.3), g.randn((out_c,))
    dy = g.randn((n, out_c, h, w))
    want_y = orc.conv2d_forward(x, wt, b, 1, 1)
    want = orc.conv2d_backward(x, wt, dy, 1, 1)
    y = pkg.conv2d(dev(x, cuda), dev(wt, cuda), dev(b, cuda), stride=1, padding=1, precision=pkg.PRECISION_TF32)
    got = pkg.conv2d_backward(dev(x, cuda), dev(wt, cuda), dev(dy, cuda), stride=1, padding=1,
                              precision=pkg.PRECISION_TF32)
    pkg.status()
    e = orc.scaled_error(y.cpu().numpy(), want_y)
    assert 1e-6 < e <= 4.0 * np.sqrt(c * k * k) * 2.0 ** -11
    positions = n * h * w
    assert orc.scaled_error(got[0].cpu().numpy(), want[0]) <= 4.0 * np.sqrt(out_c * k * k) * 2.0 ** -11 * 4
    assert orc.scaled_error(got[1].cpu().numpy(), want[1]) <= 4.0 * np.sqrt(positions) * 2.0 ** -11 * 4
    assert orc.scaled_error(got[2].cpu().numpy(), want[2]) <= 4.0 * np.sqrt(positions) * 2.0 ** -11 * 4
