"""The fused attention kernel against (a) the reference's PyTorch golden vectors
(tests/test_reference.cpp:296-340, abs 1e-4) and (b) the reference's own sequence — product against
K^T, * scale, + mask, softmax (max, exp, sequential fp32 sum, divide), product with V
(src/transformer.cpp:279-304, src/tensor_ops.cpp:621-647) — evaluated with the CPU oracle."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def dev(x, cuda):
    import torch

    return torch.from_numpy(np.ascontiguousarray(x)).to(cuda)


def reference_attention(orc, q, k, v, mask):
    lead = q.shape[:-2]
    q3, k3, v3 = (t.reshape((-1,) + t.shape[-2:]) for t in (q, k, v))
    scale = np.float32(1.0) / np.sqrt(np.float32(q.shape[-1]))
    scores = orc.matmul(q3, np.ascontiguousarray(k3.transpose(0, 2, 1))) * scale
    if mask is not None:
        scores = scores + mask
    mx = scores.max(-1, keepdims=True)
    e = np.exp(scores - mx, dtype=np.float32)
    denom = np.zeros(e.shape[:-1] + (1,), np.float32)
    for j in range(e.shape[-1]):  # sequential fp32 sum, as the reference's loop
        denom[..., 0] += e[..., j]
    w = (e / denom).astype(np.float32)
    out = orc.matmul(w, v3)
    return out.reshape(lead + out.shape[-2:]), w.reshape(lead + w.shape[-2:])


def test_pytorch_golden_attention(pkg, cuda, golden_dir):
    z = np.load(golden_dir / "pytorch_attention.npz")
    for name in ["attention", "attention_causal"]:
        mask = z[f"{name}/mask"] if f"{name}/mask" in z.files else None
        out = pkg.scaled_dot_product_attention(dev(z[f"{name}/q"], cuda), dev(z[f"{name}/k"], cuda),
                                               dev(z[f"{name}/v"], cuda), dev(mask, cuda) if mask is not None else None)
        pkg.status()
        assert np.max(np.abs(out.cpu().numpy() - z[f"{name}/output"])) <= 1e-4


@pytest.mark.parametrize("shape", [
    # (lead, s_q, s_k, d_k, d_v)
    ((32, 4), 64, 64, 24, 24),    # the char-LM configuration: 128 heads of 64 x 24
    ((2, 3), 5, 5, 4, 4),         # the reference's fixture shape
    ((3,), 128, 128, 64, 64),     # the kernel's limits
    ((5,), 17, 33, 9, 20),        # nothing aligned, s_q != s_k, d_k != d_v
    ((), 1, 1, 1, 1),
])
@pytest.mark.parametrize("causal", [False, True])
def test_against_reference_sequence(pkg, orc, cuda, shape, causal):
    lead, s_q, s_k, d_k, d_v = shape
    g = orc.Rng(70)
    q, k, v = g.randn(lead + (s_q, d_k)), g.randn(lead + (s_k, d_k)), g.randn(lead + (s_k, d_v))
    mask = None
    if causal:
        mask = np.triu(np.full((s_q, s_k), -1e9, np.float32), 1)  # make_causal_mask: 0 on and below the diagonal
    want, want_w = reference_attention(orc, q, k, v, mask)
    before = pkg.launch_count()
    out, w = pkg.scaled_dot_product_attention(dev(q, cuda), dev(k, cuda), dev(v, cuda),
                                              dev(mask, cuda) if causal else None, return_weights=True)
    pkg.status()
    assert pkg.launch_count() == before + 1, "one kernel for the whole attention core"
    assert orc.scaled_error(w.cpu().numpy(), want_w) <= 1e-5
    assert orc.scaled_error(out.cpu().numpy(), want) <= 1e-5
    rows = w.cpu().numpy().sum(-1)
    assert np.allclose(rows, 1.0, atol=1e-5)


def test_limits_are_reported_not_silently_wrong(pkg, cuda):
    import torch

    q = torch.zeros((2, 129, 8), device=cuda)
    with pytest.raises(pkg.B200Error) as err:
        pkg.scaled_dot_product_attention(q, q, q)
    assert err.value.code == -2
    with pytest.raises(ValueError):
        pkg.scaled_dot_product_attention(torch.zeros((2, 4, 8), device=cuda), torch.zeros((2, 4, 6), device=cuda),
                                         torch.zeros((2, 4, 6), device=cuda))
