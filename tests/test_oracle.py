"""Pins the CPU oracle: against the reference's own golden vectors and known answers, against
outputs of the unmodified reference engine recorded in tests/golden/, and — when the reference
build is present — against that build directly, bit for bit."""
import hashlib
import json
import sys

import numpy as np
import pytest

sys.path.insert(0, str(__import__("pathlib").Path(__file__).resolve().parent / "golden"))


def sha(x):
    return hashlib.sha256(np.ascontiguousarray(x, dtype="<f4").tobytes()).hexdigest()


def test_known_answers(orc, golden_dir):
    spec = json.loads((golden_dir / "known_answers.json").read_text())
    for case in spec["products"]:
        a = np.array(case["a"], dtype=np.float32).reshape(case["a_shape"])
        b = np.array(case["b"], dtype=np.float32).reshape(case["b_shape"])
        out = orc.matmul(a, b)
        assert list(out.shape) == case["out_shape"]
        if "out" in case:
            assert out.reshape(-1).tolist() == [float(v) for v in case["out"]]
        for idx, val in case.get("out_at", {}).items():
            assert out.reshape(-1)[int(idx)] == float(val)
    for case in spec["throws"]:
        with pytest.raises(ValueError):
            orc.matmul(np.ones(case["a_shape"], np.float32), np.ones(case["b_shape"], np.float32))


def test_pytorch_golden_vectors(orc, golden_dir):
    """Same checks and tolerance as the reference's tests/test_reference.cpp:99-114 (abs 1e-4)."""
    z = np.load(golden_dir / "pytorch_matmul.npz")
    for name in ["matmul", "matmul_batched", "matmul_shared"]:
        a, b, g = z[f"{name}/a"], z[f"{name}/b"], z[f"{name}/grad_output"]
        out = orc.matmul(a, b)
        ga, gb = orc.matmul_backward(a, b, g)
        assert np.max(np.abs(out - z[f"{name}/output"])) <= 1e-4
        assert np.max(np.abs(ga - z[f"{name}/grad.a"])) <= 1e-4
        assert np.max(np.abs(gb - z[f"{name}/grad.b"])) <= 1e-4


def test_reference_run_vectors(orc, golden_dir):
    """Bit-exact against what the unmodified reference engine produced on the same seeds."""
    import make_golden

    z = np.load(golden_dir / "reference_runs.npz")
    meta = json.loads((golden_dir / "reference_runs.json").read_text())
    for seed in (0, 1, 7):
        g = orc.Rng(seed)
        assert np.array_equal(g.rand((33,), -1.0, 1.0).view(np.uint32), z[f"rng/seed{seed}/rand"].view(np.uint32))
        assert np.array_equal(g.randn((33,), 0.5, 2.0).view(np.uint32), z[f"rng/seed{seed}/randn"].view(np.uint32))
        assert np.array_equal(g.rand((4,), 0.0, 1.0).view(np.uint32), z[f"rng/seed{seed}/rand_after"].view(np.uint32))
    for name in make_golden.CONFIGS:
        a, b = make_golden.config_inputs(name, orc.Rng)
        assert sha(a) == meta[name]["a_sha256"] and sha(b) == meta[name]["b_sha256"]
        c = orc.matmul(a, b)
        assert sha(c) == meta[name]["out_sha256"], name
        step = meta[name]["sample_step"]
        assert np.array_equal(c.reshape(-1)[::step].view(np.uint32), z[f"{name}/sample"].view(np.uint32))
        gout = orc.Rng(99).randn(c.shape)
        ga, gb = orc.matmul_backward(a, b, gout)
        assert sha(ga) == meta[name]["grad_a_sha256"], name
        assert sha(gb) == meta[name]["grad_b_sha256"], name


def test_thread_count_does_not_change_bits(orc):
    """tests/test_tensor.cpp:456-476: one row is always summed by one thread, k ascending."""
    g = orc.Rng(7)
    a, b = g.randn((200, 150)), g.randn((150, 120))
    one = orc.matmul(a, b, threads=1)
    four = orc.matmul(a, b, threads=4)
    assert np.array_equal(one.view(np.uint32), four.view(np.uint32))


def test_zero_skip_never_forms_zero_times_inf(orc):
    """The a == 0 skip (src/tensor_ops.cpp:555) means 0 x inf never becomes NaN."""
    a = np.array([[0.0, 1.0]], dtype=np.float32)
    b = np.array([[np.inf], [2.0]], dtype=np.float32)
    assert orc.matmul(a, b)[0, 0] == 2.0


def test_transposed_forms_equal_materialised_transposes(orc):
    g = orc.Rng(3)
    a = g.randn((3, 17, 23))
    b_nk = g.randn((3, 11, 23))
    a_km = g.randn((3, 23, 17))
    b = g.randn((3, 23, 11))
    assert np.array_equal(orc.matmul_nt(a, b_nk), orc.matmul(a, np.ascontiguousarray(b_nk.transpose(0, 2, 1))))
    assert np.array_equal(orc.matmul_tn(a_km, b), orc.matmul(np.ascontiguousarray(a_km.transpose(0, 2, 1)), b))


def test_fp64_product(orc):
    g = orc.Rng(5)
    a, b = g.randn((33, 65)), g.randn((65, 129))
    want = a.astype(np.float64) @ b.astype(np.float64)
    assert np.allclose(orc.matmul_f64(a, b), want, rtol=1e-13, atol=1e-13)
    assert np.allclose(orc.matmul_f64(np.ascontiguousarray(a.T), b, trans_a=True), want, rtol=1e-13, atol=1e-13)
    assert np.allclose(orc.matmul_f64(a, np.ascontiguousarray(b.T), trans_b=True), want, rtol=1e-13, atol=1e-13)


def test_against_reference_build_when_present(orc):
    """Direct bit-for-bit comparison with the unmodified reference engine (oracle/_ref)."""
    if not orc.have_ref():
        pytest.skip("oracle/_ref not built on this machine")
    g = orc.Rng(11)
    cases = [((1, 1), (1, 1)), ((17, 23), (23, 31)), ((33, 129), (129, 65)), ((4, 3, 17, 23), (4, 3, 23, 11)),
             ((8, 12, 40), (40, 20)), ((40, 12), (5, 12, 7)), ((131, 133), (133, 135))]
    for sa, sb in cases:
        a, b = g.randn(sa), g.randn(sb)
        a[a < -0.5] = 0.0  # exercise the zero-skip
        assert np.array_equal(orc.matmul(a, b).view(np.uint32), orc.ref_matmul(a, b).view(np.uint32)), (sa, sb)


def test_conv_restatement_against_golden(orc, golden_dir):
    """The numpy restatement of Conv2d forward + backward (im2col, product, bias, permute; product
    backward, col2im) reproduces, bit for bit, what the unmodified reference engine produced on the
    recorded seeded inputs, and the reference's PyTorch vectors within their 1e-4."""
    z = np.load(golden_dir / "reference_conv_backward.npz")
    for tag in ("pad1", "stride2", "k5pad2"):
        stride, pad = (int(v) for v in z[f"{tag}/window"])
        x, wt, b, dy = z[f"{tag}/x"], z[f"{tag}/weight"], z[f"{tag}/bias"], z[f"{tag}/grad_output"]
        assert np.array_equal(orc.conv2d_forward(x, wt, b, stride, pad), z[f"{tag}/output"])
        gx, gw, gb = orc.conv2d_backward(x, wt, dy, stride, pad)
        assert np.array_equal(gx, z[f"{tag}/grad.x"])
        assert np.array_equal(gw, z[f"{tag}/grad.weight"])
        assert np.array_equal(gb, z[f"{tag}/grad.bias"])
    t = np.load(golden_dir / "pytorch_conv2d.npz")
    for name, stride, pad in [("conv2d_pad1", 1, 1), ("conv2d_stride2", 2, 0)]:
        gx, gw, gb = orc.conv2d_backward(t[f"{name}/input"], t[f"{name}/weight"], t[f"{name}/grad_output"], stride, pad)
        assert np.max(np.abs(gx - t[f"{name}/grad.input"])) <= 1e-4
        assert np.max(np.abs(gw - t[f"{name}/grad.weight"])) <= 1e-4
        assert np.max(np.abs(gb - t[f"{name}/grad.bias"])) <= 1e-4


@pytest.mark.skipif(not __import__("oracle.oracle_py", fromlist=["x"]).have_ref(), reason="reference engine not built here")
def test_conv_restatement_against_reference_engine(orc):
    for (n, c, h, w, oc, k, stride, pad) in [(2, 3, 8, 8, 4, 3, 1, 1), (3, 5, 17, 13, 7, 3, 2, 0), (2, 4, 7, 9, 3, 2, 3, 1)]:
        g = orc.Rng(5)
        x, wt, b = g.randn((n, c, h, w)), g.randn((oc, c, k, k)), g.randn((oc,))
        oh, ow = (h + 2 * pad - k) // stride + 1, (w + 2 * pad - k) // stride + 1
        dy = g.randn((n, oc, oh, ow))
        y, gx, gw, gb = orc.ref_conv2d_backward(x, wt, b, dy, stride, pad)
        assert np.array_equal(orc.conv2d_forward(x, wt, b, stride, pad), y)
        gx2, gw2, gb2 = orc.conv2d_backward(x, wt, dy, stride, pad)
        assert np.array_equal(gx, gx2) and np.array_equal(gw, gw2) and np.array_equal(gb, gb2)


def test_attention_restatement_against_golden(orc, golden_dir):
    """The restatement of scaled_dot_product_attention and its backward reproduces, bit for bit, the
    recorded results of the unmodified reference engine, and the reference's PyTorch vectors within 1e-4."""
    import make_golden

    z = np.load(golden_dir / "reference_attention_backward.npz")
    for tag in make_golden.ATTENTION_BACKWARD_CASES:
        q, k, v, go, mask = make_golden.attention_backward_inputs(tag, orc.Rng)
        out, _, gq, gk, gv = orc.attention_backward(q, k, v, mask, go)
        assert np.array_equal(out, z[f"{tag}/output"])
        assert np.array_equal(gq, z[f"{tag}/grad.q"])
        assert np.array_equal(gk, z[f"{tag}/grad.k"])
        assert np.array_equal(gv, z[f"{tag}/grad.v"])
    t = np.load(golden_dir / "pytorch_attention.npz")
    for name in ["attention", "attention_causal"]:
        mask = t[f"{name}/mask"] if f"{name}/mask" in t.files else None
        flat = lambda a: a.reshape((-1,) + a.shape[-2:])  # noqa: E731
        out, w, gq, gk, gv = orc.attention_backward(flat(t[f"{name}/q"]), flat(t[f"{name}/k"]), flat(t[f"{name}/v"]),
                                                    mask, flat(t[f"{name}/grad_output"]))
        for got, key in ((out, "output"), (w, "weights"), (gq, "grad.q"), (gk, "grad.k"), (gv, "grad.v")):
            assert np.max(np.abs(got - flat(t[f"{name}/{key}"]))) <= 1e-4
