"""The fused attention backward kernel — scores recomputed, five tensor-core products and the softmax
backward in one launch — against (a) the reference's PyTorch golden gradients
(tests/test_reference.cpp:296-320, abs 1e-4), (b) recorded results of the unmodified reference engine's
own attention + autograd, and (c) the reference's sequence of backward steps (src/transformer.cpp:279-304,
src/tensor_ops.cpp:570-585, 649-668) evaluated with the CPU oracle on seeded inputs."""
import sys
from pathlib import Path

import numpy as np
import pytest

sys.path.insert(0, str(Path(__file__).resolve().parent / "golden"))

pytestmark = pytest.mark.gpu


def dev(x, cuda):
    import torch

    return torch.from_numpy(np.ascontiguousarray(x)).to(cuda)


def test_pytorch_golden_attention_gradients(pkg, cuda, golden_dir):
    z = np.load(golden_dir / "pytorch_attention.npz")
    for name in ["attention", "attention_causal"]:
        mask = dev(z[f"{name}/mask"], cuda) if f"{name}/mask" in z.files else None
        before = pkg.launch_count()
        gq, gk, gv = pkg.scaled_dot_product_attention_backward(
            dev(z[f"{name}/q"], cuda), dev(z[f"{name}/k"], cuda), dev(z[f"{name}/v"], cuda),
            dev(z[f"{name}/grad_output"], cuda), mask)
        pkg.status()
        assert pkg.launch_count() == before + 1, "one kernel for the whole backward of the attention core"
        assert np.max(np.abs(gq.cpu().numpy() - z[f"{name}/grad.q"])) <= 1e-4
        assert np.max(np.abs(gk.cpu().numpy() - z[f"{name}/grad.k"])) <= 1e-4
        assert np.max(np.abs(gv.cpu().numpy() - z[f"{name}/grad.v"])) <= 1e-4


def test_recorded_reference_engine_gradients(pkg, orc, cuda, golden_dir):
    import make_golden

    z = np.load(golden_dir / "reference_attention_backward.npz")
    for tag in make_golden.ATTENTION_BACKWARD_CASES:
        q, k, v, go, mask = make_golden.attention_backward_inputs(tag, orc.Rng)
        gq, gk, gv = pkg.scaled_dot_product_attention_backward(dev(q, cuda), dev(k, cuda), dev(v, cuda), dev(go, cuda),
                                                               dev(mask, cuda) if mask is not None else None)
        pkg.status()
        assert orc.scaled_error(gq.cpu().numpy(), z[f"{tag}/grad.q"]) <= 1e-5
        assert orc.scaled_error(gk.cpu().numpy(), z[f"{tag}/grad.k"]) <= 1e-5
        assert orc.scaled_error(gv.cpu().numpy(), z[f"{tag}/grad.v"]) <= 1e-5


@pytest.mark.parametrize("shape", [
    # (lead, s_q, s_k, d_k, d_v)
    ((32, 4), 64, 64, 24, 24),    # the char-LM configuration: 128 heads of 64 x 24
    ((2, 3), 5, 5, 4, 4),         # the reference's fixture shape
    ((3,), 64, 64, 64, 64),       # the widest heads that fit at S = 64
    ((5,), 17, 33, 9, 20),        # nothing aligned, s_q != s_k, d_k != d_v
    ((2,), 40, 72, 16, 8),        # three 32-column groups of keys
    ((4,), 8, 128, 32, 32),       # few queries over the longest key axis
    ((7, 61), 16, 24, 8, 8),      # 427 heads: every CTA walks several heads
    ((), 1, 1, 1, 1),
])
@pytest.mark.parametrize("causal", [False, True])
def test_against_reference_sequence(pkg, orc, cuda, shape, causal):
    lead, s_q, s_k, d_k, d_v = shape
    g = orc.Rng(80)
    q, k, v = g.randn(lead + (s_q, d_k)), g.randn(lead + (s_k, d_k)), g.randn(lead + (s_k, d_v))
    go = g.randn(lead + (s_q, d_v))
    mask = np.triu(np.full((s_q, s_k), -1e9, np.float32), 1) if causal else None
    flat = lambda t: t.reshape((-1,) + t.shape[-2:])  # noqa: E731
    _, _, want_q, want_k, want_v = orc.attention_backward(flat(q), flat(k), flat(v), mask, flat(go))
    gq, gk, gv = pkg.scaled_dot_product_attention_backward(dev(q, cuda), dev(k, cuda), dev(v, cuda), dev(go, cuda),
                                                           dev(mask, cuda) if causal else None)
    pkg.status()
    tol = 2e-5  # two products deep
    assert orc.scaled_error(flat(gq.cpu().numpy()), want_q) <= tol
    assert orc.scaled_error(flat(gk.cpu().numpy()), want_k) <= tol
    assert orc.scaled_error(flat(gv.cpu().numpy()), want_v) <= tol


def test_heads_by_strides_equal_permuted_copies(pkg, cuda, orc):
    """Gradients of the projections (B, S, H*hd) through the strided entry point equal, bit for bit, the
    contiguous entry point's on materialised (B, H, S, hd) copies, merged back."""
    import torch

    b, heads, s, hd = 4, 4, 64, 24
    g = orc.Rng(81)
    q, k, v, go = (dev(g.randn((b, s, heads * hd)), cuda) for _ in range(4))
    mask = torch.triu(torch.full((s, s), -1e9, device=cuda), 1)
    gq, gk, gv = pkg.multi_head_attention_core_backward(q, k, v, go, heads, mask)
    pkg.status()
    split = lambda t: t.reshape(b, s, heads, hd).permute(0, 2, 1, 3).contiguous()  # noqa: E731
    merge = lambda t: t.permute(0, 2, 1, 3).reshape(b, s, heads * hd)  # noqa: E731
    wq, wk, wv = pkg.scaled_dot_product_attention_backward(split(q), split(k), split(v), split(go), mask)
    pkg.status()
    assert torch.equal(gq, merge(wq)) and torch.equal(gk, merge(wk)) and torch.equal(gv, merge(wv))
    # column slices of one fused Q|K|V tensor
    qkv = dev(g.randn((b, s, 3 * heads * hd)), cuda)
    dm = heads * hd
    sq, sk, sv = qkv[:, :, :dm], qkv[:, :, dm:2 * dm], qkv[:, :, 2 * dm:]
    a = pkg.multi_head_attention_core_backward(sq, sk, sv, go, heads, mask)
    c = pkg.multi_head_attention_core_backward(sq.contiguous(), sk.contiguous(), sv.contiguous(), go, heads, mask)
    pkg.status()
    for x, y in zip(a, c):
        assert torch.equal(x, y)


def test_accumulates_and_skips(pkg, orc, cuda):
    """beta = 1 adds into existing gradients (Tensor::add_grad); NULL outputs are skipped."""
    import torch

    g = orc.Rng(82)
    q, k, v, go = (dev(g.randn((6, 32, 16)), cuda) for _ in range(4))
    gq, gk, gv = pkg.scaled_dot_product_attention_backward(q, k, v, go)
    acc_q, acc_v = gq.clone(), gv.clone()
    pkg.lib.attention_backward_strided(q, k, v, None, go, acc_q, None, acc_v, batch=6, heads=1, s_q=32, s_k=32, d_k=16,
                                       d_v=16, q_strides=(512, 0, 16), k_strides=(512, 0, 16), v_strides=(512, 0, 16),
                                       out_strides=(512, 0, 16), scale=0.25, beta=1.0)
    pkg.status()
    assert torch.allclose(acc_q, 2 * gq, rtol=1e-6, atol=1e-6)
    assert torch.allclose(acc_v, 2 * gv, rtol=1e-6, atol=1e-6)


def test_limits_are_refused_not_faked(pkg, cuda):
    import torch

    big = torch.zeros((2, 128, 64), device=cuda)
    with pytest.raises(pkg.B200Error) as err:  # the tiles of S = 128, d = 64 do not fit one CTA: the fused
        pkg.lib.attention_backward_strided(     # kernel's own entry point says so
            big, big, big, None, big, big.clone(), big.clone(), big.clone(), batch=2, heads=1, s_q=128, s_k=128,
            d_k=64, d_v=64, q_strides=(8192, 0, 64), k_strides=(8192, 0, 64), v_strides=(8192, 0, 64),
            out_strides=(8192, 0, 64), scale=0.125)
    assert err.value.code == -2
    with pytest.raises(ValueError):
        pkg.scaled_dot_product_attention_backward(big, big, big, torch.zeros((2, 128, 32), device=cuda))


def test_tf32_mode_is_coarser_but_close(pkg, orc, cuda):
    """The opt-in single-product TF32 mode of the forward and backward attention kernels: same code path
    without the correction products — about three decimal digits."""
    g = orc.Rng(83)
    lead, s, d = 6, 64, 24
    q, k, v, go = g.randn((lead, s, d)), g.randn((lead, s, d)), g.randn((lead, s, d)), g.randn((lead, s, d))
    out_want, _, want_q, want_k, want_v = orc.attention_backward(q, k, v, None, go)
    out = pkg.scaled_dot_product_attention(dev(q, cuda), dev(k, cuda), dev(v, cuda), precision=pkg.PRECISION_TF32)
    gq, gk, gv = pkg.scaled_dot_product_attention_backward(dev(q, cuda), dev(k, cuda), dev(v, cuda), dev(go, cuda),
                                                           precision=pkg.PRECISION_TF32)
    pkg.status()
    e_out = orc.scaled_error(out.cpu().numpy(), out_want)
    assert 1e-6 < e_out <= 2e-2
    for got, want in ((gq, want_q), (gk, want_k), (gv, want_v)):
        assert orc.scaled_error(got.cpu().numpy(), want) <= 5e-2
