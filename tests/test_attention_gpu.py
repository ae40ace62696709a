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
    ((7, 61), 16, 24, 8, 8),      # 427 heads: every CTA walks several heads
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
    out = torch.empty((2, 129, 8), device=cuda)
    with pytest.raises(pkg.B200Error) as err:  # the fused kernel's own entry point keeps its limits
        pkg.lib.attention_forward(q, q, q, None, out, None, batch=2, s_q=129, s_k=129, d_k=8, d_v=8, scale=1.0)
    assert err.value.code == -2
    with pytest.raises(pkg.B200Error) as err:  # the any-size entry point without the scratch it asks for
        pkg.attention_any(q, q, q, None, out, None, batch=2, heads=1, s_q=129, s_k=129, d_k=8, d_v=8,
                          q_strides=(129 * 8, 0, 8), k_strides=(129 * 8, 0, 8), v_strides=(129 * 8, 0, 8),
                          out_strides=(129 * 8, 0, 8), scale=1.0)
    assert err.value.code == -3
    with pytest.raises(ValueError):
        pkg.scaled_dot_product_attention(torch.zeros((2, 4, 8), device=cuda), torch.zeros((2, 4, 6), device=cuda),
                                         torch.zeros((2, 4, 6), device=cuda))


# ---------------------------------------------------------------------------------------------
# Heads addressed through strides: MultiHeadAttention::forward without its permute copies
# (src/transformer.cpp:339-357)
# ---------------------------------------------------------------------------------------------

def split_heads(t, heads):
    b, s, dm = t.shape
    return np.ascontiguousarray(t.reshape(b, s, heads, dm // heads).transpose(0, 2, 1, 3))


@pytest.mark.parametrize("dims", [
    # (batch, heads, s_q, s_k, head_dim)
    (32, 4, 64, 64, 24),   # the char-LM block
    (2, 2, 5, 5, 4),       # the reference's MultiHeadAttention(8, 2) fixture shape
    (3, 5, 17, 33, 9),     # nothing aligned
    (1, 1, 128, 128, 64),  # the kernel's limits
])
@pytest.mark.parametrize("causal", [False, True])
def test_strided_heads_equal_permuted_copies(pkg, cuda, orc, dims, causal):
    """The strided entry point on (B, S, H*hd) projections gives, bit for bit, what the contiguous entry
    point gives on the materialised (B, H, S, hd) permutes, merged back — and both match the reference's
    sequence."""
    b, heads, s_q, s_k, hd = dims
    g = orc.Rng(71)
    q, k, v = g.randn((b, s_q, heads * hd)), g.randn((b, s_k, heads * hd)), g.randn((b, s_k, heads * hd))
    mask = np.triu(np.full((s_q, s_k), -1e9, np.float32), 1) if causal else None
    dmask = dev(mask, cuda) if causal else None
    before = pkg.launch_count()
    merged, w = pkg.multi_head_attention_core(dev(q, cuda), dev(k, cuda), dev(v, cuda), heads, dmask,
                                              return_weights=True)
    pkg.status()
    assert pkg.launch_count() == before + 1
    out4, w4 = pkg.scaled_dot_product_attention(dev(split_heads(q, heads), cuda), dev(split_heads(k, heads), cuda),
                                                dev(split_heads(v, heads), cuda), dmask, return_weights=True)
    pkg.status()
    want_merged = out4.permute(0, 2, 1, 3).reshape(b, s_q, heads * hd)
    assert np.array_equal(merged.cpu().numpy(), want_merged.cpu().numpy())
    assert np.array_equal(w.cpu().numpy(), w4.cpu().numpy())
    ref_out, _ = reference_attention(orc, split_heads(q, heads), split_heads(k, heads), split_heads(v, heads), mask)
    ref_merged = ref_out.transpose(0, 2, 1, 3).reshape(b, s_q, heads * hd)
    assert orc.scaled_error(merged.cpu().numpy(), ref_merged) <= 1e-5


def test_strided_heads_on_fused_qkv_slices(pkg, cuda, orc):
    """q, k and v as column slices of ONE (B, S, 3*d_model) product (row stride 3*d_model)."""
    import torch

    b, heads, s, hd = 4, 4, 64, 24
    dm = heads * hd
    g = orc.Rng(72)
    qkv = dev(g.randn((b, s, 3 * dm)), cuda)
    q, k, v = qkv[:, :, :dm], qkv[:, :, dm:2 * dm], qkv[:, :, 2 * dm:]
    got = pkg.multi_head_attention_core(q, k, v, heads)
    pkg.status()
    want = pkg.multi_head_attention_core(q.contiguous(), k.contiguous(), v.contiguous(), heads)
    pkg.status()
    assert torch.equal(got, want)


def test_pytorch_golden_multihead(pkg, cuda, golden_dir):
    """The reference's PyTorch vectors for a whole MultiHeadAttention(8, 2) forward
    (tests/test_reference.cpp:322-339, abs 1e-4): four Linear layers around the strided core."""
    z = np.load(golden_dir / "pytorch_multihead.npz")
    x = dev(z["input"], cuda)
    proj = {}
    for tag in ("query", "key", "value"):
        proj[tag] = pkg.linear(x, dev(z[f"w.{tag}.weight"], cuda), dev(z[f"w.{tag}.bias"].reshape(-1), cuda))
    merged = pkg.multi_head_attention_core(proj["query"], proj["key"], proj["value"], 2)
    out = pkg.linear(merged, dev(z["w.out.weight"], cuda), dev(z["w.out.bias"].reshape(-1), cuda))
    pkg.status()
    assert np.max(np.abs(out.cpu().numpy() - z["output"])) <= 1e-4


def test_strided_argument_errors(pkg, cuda):
    import torch

    x = torch.zeros((2, 8, 12), device=cuda)
    with pytest.raises(ValueError):
        pkg.multi_head_attention_core(x, x, x, 5)              # d_model not divisible by heads
    with pytest.raises(ValueError):
        pkg.multi_head_attention_core(x, x[:, :, :8], x, 2)    # query/key widths differ
    with pytest.raises(ValueError):
        pkg.multi_head_attention_core(x[0], x[0], x[0], 2)     # not (batch, seq, d_model)
    with pytest.raises(ValueError):
        pkg.multi_head_attention_core(x.transpose(1, 2), x.transpose(1, 2), x.transpose(1, 2), 2)  # last axis strided
