"""Attention for heads beyond the fused kernels' tiles (the reference's scaled_dot_product_attention takes
any S and d, src/transformer.cpp:279-304): the any-size entry points run them composed on the device —
scores product with scale and mask in its store, an owned row-softmax kernel, weights x v; backward
through the transposed forms and one softmax-backward row kernel — and are checked against the
reference's sequence of steps evaluated by the CPU oracle, forward and gradients."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def dev(x, cuda):
    import torch

    return torch.from_numpy(np.ascontiguousarray(x)).to(cuda)


CASES = [
    # (lead, s_q, s_k, d_k, d_v)
    ((2,), 128, 128, 64, 64),   # forward fused, backward composed (the tiles of S = 128 do not fit one CTA)
    ((3,), 256, 256, 64, 64),
    ((2, 2), 512, 512, 128, 128),
    ((2,), 130, 257, 72, 40),   # nothing aligned, s_q != s_k, d_k != d_v
]


@pytest.mark.parametrize("shape", CASES)
@pytest.mark.parametrize("causal", [False, True])
def test_forward_and_gradients_against_the_reference_sequence(pkg, orc, cuda, shape, causal):
    lead, s_q, s_k, d_k, d_v = shape
    g = orc.Rng(90)
    q, k, v = g.randn(lead + (s_q, d_k)), g.randn(lead + (s_k, d_k)), g.randn(lead + (s_k, d_v))
    go = g.randn(lead + (s_q, d_v))
    mask = np.triu(np.full((s_q, s_k), -1e9, np.float32), 1) if causal else None
    flat = lambda t: t.reshape((-1,) + t.shape[-2:])  # noqa: E731
    want_out, want_w, want_q, want_k, want_v = orc.attention_backward(flat(q), flat(k), flat(v), mask, flat(go))
    Q, K, V, GO = dev(q, cuda), dev(k, cuda), dev(v, cuda), dev(go, cuda)
    M = dev(mask, cuda) if causal else None
    out, w = pkg.scaled_dot_product_attention(Q, K, V, M, return_weights=True)
    out2 = pkg.scaled_dot_product_attention(Q, K, V, M)  # without a weights buffer: the scratch path
    gq, gk, gv = pkg.scaled_dot_product_attention_backward(Q, K, V, GO, M)
    pkg.status()
    # scores have magnitude sqrt(d_k) before the scale and d_k-long contractions behind them
    tol = max(2e-5, orc.parity_tolerance(max(s_k, d_k)))
    assert orc.scaled_error(flat(w.cpu().numpy()), want_w) <= tol
    assert np.allclose(w.cpu().numpy().sum(-1), 1.0, atol=1e-5)
    assert orc.scaled_error(flat(out.cpu().numpy()), want_out) <= tol
    assert np.array_equal(out.cpu().numpy(), out2.cpu().numpy())
    for got, want in ((gq, want_q), (gk, want_k), (gv, want_v)):
        assert orc.scaled_error(flat(got.cpu().numpy()), want) <= 2 * tol


def test_heads_by_strides_equal_permuted_copies_large(pkg, orc, cuda):
    """(B, S, H * hd) projections with S = 256: the composed path addresses heads by strides too (one launch
    per batch element over its heads) and equals the contiguous path on materialised (B, H, S, hd) copies."""
    import torch

    b, heads, s, hd = 2, 4, 256, 32
    g = orc.Rng(91)
    q, k, v, go = (dev(g.randn((b, s, heads * hd)), cuda) for _ in range(4))
    mask = torch.triu(torch.full((s, s), -1e9, device=cuda), 1)
    merged = pkg.multi_head_attention_core(q, k, v, heads, mask)
    gq, gk, gv = pkg.multi_head_attention_core_backward(q, k, v, go, heads, mask)
    pkg.status()
    split = lambda t: t.reshape(b, s, heads, hd).permute(0, 2, 1, 3).contiguous()  # noqa: E731
    merge = lambda t: t.permute(0, 2, 1, 3).reshape(b, s, heads * hd)  # noqa: E731
    want = pkg.scaled_dot_product_attention(split(q), split(k), split(v), mask)
    wq, wk, wv = pkg.scaled_dot_product_attention_backward(split(q), split(k), split(v), split(go), mask)
    pkg.status()
    assert torch.equal(merged, merge(want))
    assert torch.equal(gq, merge(wq)) and torch.equal(gk, merge(wk)) and torch.equal(gv, merge(wv))


def test_accumulation_and_workspace_contract(pkg, orc, cuda):
    import torch

    g = orc.Rng(92)
    b, s, d = 2, 200, 48
    q, k, v, go = (dev(g.randn((b, s, d)), cuda) for _ in range(4))
    gq, gk, gv = pkg.scaled_dot_product_attention_backward(q, k, v, go)
    need = pkg.attention_any_workspace(batch=b, heads=1, s_q=s, s_k=s, d_k=d, d_v=d, backward=True)
    assert need == 2 * b * s * s * 4
    assert pkg.attention_any_workspace(batch=b, heads=1, s_q=64, s_k=64, d_k=24, d_v=24, backward=True) == 0
    ws = torch.empty(need, dtype=torch.uint8, device=cuda)
    st = (s * d, 0, d)
    acc_q, acc_k, acc_v = gq.clone(), gk.clone(), gv.clone()
    pkg.attention_backward_any(q, k, v, None, go, acc_q, acc_k, acc_v, batch=b, heads=1, s_q=s, s_k=s, d_k=d, d_v=d,
                               q_strides=st, k_strides=st, v_strides=st, out_strides=st, scale=d ** -0.5, beta=1.0,
                               workspace=ws, workspace_bytes=need)
    pkg.status()
    for acc, once in ((acc_q, gq), (acc_k, gk), (acc_v, gv)):
        assert torch.allclose(acc, 2 * once, rtol=1e-6, atol=1e-6)
    with pytest.raises(pkg.B200Error) as err:
        pkg.attention_backward_any(q, k, v, None, go, acc_q, acc_k, acc_v, batch=b, heads=1, s_q=s, s_k=s, d_k=d,
                                   d_v=d, q_strides=st, k_strides=st, v_strides=st, out_strides=st, scale=1.0,
                                   workspace=ws, workspace_bytes=need - 16)
    assert err.value.code == -3
