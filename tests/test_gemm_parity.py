"""GPU parity: the CUDA path, called through the C ABI, against the CPU oracle on the same
seeded inputs.  Error metric and tolerances are the reference's own
(tests/test_cuda_parity.cpp:62-137, 304-315): max |got - want| / max(1, |want|) <= 1e-5, widened
to 2K/2^24 for long contractions because the CPU loop's sequential fp32 sum drifts with K.
Integer-valued inputs must match exactly."""
import json
import sys
from pathlib import Path

import numpy as np
import pytest

sys.path.insert(0, str(Path(__file__).resolve().parent / "golden"))

pytestmark = pytest.mark.gpu


def dev(x, cuda):
    import torch

    return torch.from_numpy(np.ascontiguousarray(x)).to(cuda)


def run_matmul(pkg, cuda, a, b):
    before = pkg.launch_count()
    out = pkg.matmul(dev(a, cuda), dev(b, cuda))
    pkg.status()
    assert pkg.launch_count() > before, "no kernel was launched"  # test_cuda_parity.cpp:80-85
    return out.cpu().numpy()


def gemm(pkg, cuda, A, B, C, **kw):
    import torch

    ws_bytes = kw.pop("ws_bytes", None)
    if ws_bytes is None:
        ws_bytes = pkg.workspace_bytes(kw["batch"], kw["M"], kw["N"], kw["K"])
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=cuda)
    pkg.gemm(A, B, C, workspace=ws, workspace_bytes=ws_bytes, **kw)
    pkg.status()


# the reference's own CPU/GPU parity shape list (tests/test_cuda_parity.cpp:192-247)
REFERENCE_SHAPES = [
    ((1, 1), (1, 1)), ((17, 23), (23, 31)), ((32, 32), (32, 32)), ((33, 129), (129, 65)),
    ((127, 129), (129, 128)), ((128, 128), (128, 128)), ((129, 257), (257, 256)),
    ((256, 256), (256, 260)), ((4, 3, 17, 23), (4, 3, 23, 11)), ((8, 12, 40), (40, 20)),
    ((131, 135), (135, 133)), ((40, 12), (5, 12, 7)),
]


@pytest.mark.parametrize("sa,sb", REFERENCE_SHAPES)
def test_reference_parity_shapes(pkg, orc, cuda, sa, sb):
    g = orc.Rng(42)
    a, b = g.randn(sa), g.randn(sb)
    want = orc.matmul(a, b)
    got = run_matmul(pkg, cuda, a, b)
    assert got.shape == want.shape
    assert orc.scaled_error(got, want) <= orc.parity_tolerance(sa[-1])
    orc.assert_no_further_from_fp64(got, want, np.matmul(a.astype(np.float64), b.astype(np.float64)))


@pytest.mark.parametrize("sa,sb", REFERENCE_SHAPES)
def test_exact_on_small_integers(pkg, orc, cuda, sa, sb):
    """Inputs in [-4, 4] x [-3, 3] are exact in TF32 and every partial sum is exact in fp32,
    so any indexing, layout or remainder mistake shows as a non-zero difference
    (tests/test_cuda_parity.cpp:344-363, 432-475)."""
    rng = np.random.default_rng(7)
    a = rng.integers(-4, 5, size=sa).astype(np.float32)
    b = rng.integers(-3, 4, size=sb).astype(np.float32)
    want = orc.matmul(a, b)
    assert np.array_equal(run_matmul(pkg, cuda, a, b), want)


@pytest.mark.parametrize("M,K,N", [(9, 6272, 16), (144, 1568, 32), (144, 12544, 32), (7, 5000, 5)])
def test_split_k_shapes(pkg, orc, cuda, M, K, N):
    """The reference's tall-thin products (tests/test_cuda_parity.cpp:304-333)."""
    g = orc.Rng(9)
    a, b = g.randn((M, K)), g.randn((K, N))
    assert pkg.workspace_bytes(1, M, N, K) > 0, "expected the split-K path for this shape"
    got = run_matmul(pkg, cuda, a, b)
    want = orc.matmul(a, b)
    assert orc.scaled_error(got, want) <= orc.parity_tolerance(K)
    # the wide bound is for the CPU loop's drift over a long K; the kernel itself is held to fp64
    orc.assert_no_further_from_fp64(got, want, a.astype(np.float64) @ b.astype(np.float64))
    rng = np.random.default_rng(3)
    ai = rng.integers(-2, 3, size=(M, K)).astype(np.float32)
    bi = rng.integers(-2, 3, size=(K, N)).astype(np.float32)
    assert np.array_equal(run_matmul(pkg, cuda, ai, bi), orc.matmul(ai, bi))


def test_split_k_is_deterministic_and_optional(pkg, orc, cuda):
    import torch

    g = orc.Rng(10)
    a, b = g.randn((96, 2048)), g.randn((2048, 384))
    A, B = dev(a, cuda), dev(b, cuda)
    outs = []
    for _ in range(3):
        C = torch.empty((96, 384), device=cuda)
        gemm(pkg, cuda, A, B, C, batch=1, M=96, N=384, K=2048, lda=2048, ldb=384, ldc=384)
        outs.append(C.cpu().numpy())
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[1], outs[2])
    C = torch.empty((96, 384), device=cuda)
    gemm(pkg, cuda, A, B, C, batch=1, M=96, N=384, K=2048, lda=2048, ldb=384, ldc=384, ws_bytes=0)
    want = orc.matmul(a, b)
    assert orc.scaled_error(C.cpu().numpy(), want) <= orc.parity_tolerance(2048)
    assert orc.scaled_error(outs[0], want) <= orc.parity_tolerance(2048)


def test_beta_accumulates_onto_nonzero_destination(pkg, orc, cuda):
    """out = a x b + beta * out (tests/test_cuda_parity.cpp:263-290)."""
    g = orc.Rng(12)
    a, b, c0 = g.randn((65, 70)), g.randn((70, 36)), g.randn((65, 36))
    C = dev(c0, cuda)
    assert pkg.ops_matmul(dev(a, cuda), dev(b, cuda), C, 1, 65, 70, 36, False, False, 1.0)
    pkg.status()
    want = orc.matmul(a, b) + c0
    assert orc.scaled_error(C.cpu().numpy(), want) <= 1e-5


def test_beta_zero_ignores_garbage_in_destination(pkg, orc, cuda):
    import torch

    g = orc.Rng(13)
    a, b = g.randn((40, 24)), g.randn((24, 52))
    C = torch.full((40, 52), float("nan"), device=cuda)
    pkg.ops_matmul(dev(a, cuda), dev(b, cuda), C, 1, 40, 24, 52, False, False, 0.0)
    pkg.status()
    assert orc.scaled_error(C.cpu().numpy(), orc.matmul(a, b)) <= 1e-5


@pytest.mark.parametrize("form", ["NT", "TN", "TT"])
@pytest.mark.parametrize("M,K,N", [(64, 24, 64), (130, 45, 121), (300, 100, 520), (2048, 96, 384)])
def test_transposed_forms_match_materialised_transposes(pkg, orc, cuda, form, M, K, N):
    """The layout-descriptor forms give what the reference gets by transposing first."""
    import torch

    g = orc.Rng(14)
    tA, tB = form[0] == "T", form[1] == "T"
    a = g.randn((K, M) if tA else (M, K))
    b = g.randn((N, K) if tB else (K, N))
    opa = np.ascontiguousarray(a.T) if tA else a
    opb = np.ascontiguousarray(b.T) if tB else b
    want = orc.matmul(opa, opb)
    C = torch.empty((M, N), device=cuda)
    gemm(pkg, cuda, dev(a, cuda), dev(b, cuda), C, batch=1, M=M, N=N, K=K, transA=tA, transB=tB,
         lda=a.shape[1], ldb=b.shape[1], ldc=N)
    assert orc.scaled_error(C.cpu().numpy(), want) <= orc.parity_tolerance(K)
    orc.assert_no_further_from_fp64(C.cpu().numpy(), want, opa.astype(np.float64) @ opb.astype(np.float64))


def test_sentinel_padding_stays_untouched(pkg, orc, cuda):
    """Leading dimensions larger than the row: the gap columns keep their sentinel
    (the reference replays its index algebra against a -12345 fill, tests/test_cuda_indexing.cpp)."""
    import torch

    g = orc.Rng(15)
    M, K, N, pad = 77, 52, 45, 7
    a = np.full((M, K + pad), -12345.0, np.float32)
    b = np.full((K, N + pad), -12345.0, np.float32)
    a[:, :K], b[:, :N] = g.randn((M, K)), g.randn((K, N))
    C = torch.full((M, N + pad), -12345.0, device=cuda)
    gemm(pkg, cuda, dev(a, cuda), dev(b, cuda), C, batch=1, M=M, N=N, K=K, lda=K + pad, ldb=N + pad,
         ldc=N + pad)
    c = C.cpu().numpy()
    assert np.all(c[:, N:] == -12345.0)
    assert orc.scaled_error(c[:, :N], orc.matmul(a[:, :K].copy(), b[:, :N].copy())) <= 1e-5


@pytest.mark.parametrize("tile_n", [32, 64, 128, 256])
@pytest.mark.parametrize("loader", ["tma", "ldg"])
def test_every_tile_config_and_loader(pkg, orc, cuda, tile_n, loader):
    rng = np.random.default_rng(tile_n)
    a = rng.integers(-4, 5, size=(300, 100)).astype(np.float32)
    b = rng.integers(-3, 4, size=(100, 520)).astype(np.float32)
    pkg.set_option("tile_n", tile_n)
    pkg.set_option("force_ldg", 1 if loader == "ldg" else 0)
    try:
        got = run_matmul(pkg, cuda, a, b)
    finally:
        pkg.set_option("tile_n", 0)
        pkg.set_option("force_ldg", 0)
    assert np.array_equal(got, orc.matmul(a, b))


@pytest.mark.parametrize("form", ["NN", "NT", "TN", "TT"])
@pytest.mark.parametrize("M,K,N", [(256, 32, 256), (300, 100, 520), (770, 260, 1000)])
def test_cta_pair_kernel_exact(pkg, orc, cuda, form, M, K, N):
    """The 256 x 256 CTA-pair kernel, forced on for shapes the planner would give to the
    single-CTA kernel: integer inputs must come out exactly, in every transposition."""
    import torch

    rng = np.random.default_rng(M + N)
    tA, tB = form[0] == "T", form[1] == "T"
    a = rng.integers(-4, 5, size=(K, M) if tA else (M, K)).astype(np.float32)
    b = rng.integers(-3, 4, size=(N, K) if tB else (K, N)).astype(np.float32)
    want = orc.matmul(np.ascontiguousarray(a.T) if tA else a, np.ascontiguousarray(b.T) if tB else b)
    C = torch.full((M, N), float("nan"), device=cuda)
    pkg.set_option("pair_mode", 2)
    try:
        gemm(pkg, cuda, dev(a, cuda), dev(b, cuda), C, batch=1, M=M, N=N, K=K, transA=tA, transB=tB,
             lda=a.shape[1], ldb=b.shape[1], ldc=N)
    finally:
        pkg.set_option("pair_mode", 0)
    assert np.array_equal(C.cpu().numpy(), want)


def test_pair_and_single_kernels_agree_bitwise(pkg, orc, cuda):
    """Both kernels sum every output element in the same order (k-blocks of 32, correction
    products first), so their results are identical, not merely close."""
    import torch

    g = orc.Rng(31)
    M, K, N = 512, 384, 768
    A, B = dev(g.randn((M, K)), cuda), dev(g.randn((K, N)), cuda)
    outs = []
    for mode in (1, 2):
        pkg.set_option("pair_mode", mode)
        pkg.set_option("split_k", 1)  # no K-split: its reduction adds the parts in another order
        try:
            C = torch.empty((M, N), device=cuda)
            gemm(pkg, cuda, A, B, C, batch=1, M=M, N=N, K=K, lda=K, ldb=N, ldc=N)
            outs.append(C)
        finally:
            pkg.set_option("pair_mode", 0)
            pkg.set_option("split_k", 0)
    assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize("beta", [0.0, 1.0])
def test_tail_wave_split(pkg, orc, cuda, beta):
    """80 pair tiles on 74 clusters: the 6 tiles of the last wave run split four ways along K in a
    second launch and are reduced in a fixed order.  Exact on integers, deterministic, and equal
    within tolerance to the unsplit plan."""
    import torch

    M, N, K = 2560, 2048, 1024
    ws_bytes = pkg.workspace_bytes(1, M, N, K)
    assert ws_bytes > 0, "expected the tail-wave plan for this shape"
    rng = np.random.default_rng(5)
    a = rng.integers(-4, 5, size=(M, K)).astype(np.float32)
    b = rng.integers(-3, 4, size=(K, N)).astype(np.float32)
    c0 = rng.integers(-5, 6, size=(M, N)).astype(np.float32)
    want = orc.matmul(a, b) + beta * c0
    A, B = dev(a, cuda), dev(b, cuda)
    outs = []
    for _ in range(2):
        C = dev(c0, cuda)
        gemm(pkg, cuda, A, B, C, batch=1, M=M, N=N, K=K, lda=K, ldb=N, ldc=N, beta=beta, ws_bytes=ws_bytes)
        outs.append(C.cpu().numpy())
    assert np.array_equal(outs[0], want) and np.array_equal(outs[0], outs[1])
    g = orc.Rng(6)
    ar, br = g.randn((M, K)), g.randn((K, N))
    Ar, Br = dev(ar, cuda), dev(br, cuda)
    C1 = torch.empty((M, N), device=cuda)
    C2 = torch.empty((M, N), device=cuda)
    gemm(pkg, cuda, Ar, Br, C1, batch=1, M=M, N=N, K=K, lda=K, ldb=N, ldc=N, ws_bytes=ws_bytes)
    gemm(pkg, cuda, Ar, Br, C2, batch=1, M=M, N=N, K=K, lda=K, ldb=N, ldc=N, ws_bytes=0)
    wantr = orc.matmul(ar, br)
    assert orc.scaled_error(C1.cpu().numpy(), wantr) <= orc.parity_tolerance(K)
    # two summation orders of the same fp32 sum: each is within the K-dependent bound of the truth
    assert orc.scaled_error(C1.cpu().numpy(), C2.cpu().numpy()) <= orc.parity_tolerance(K)


def test_golden_pytorch_vectors_forward(pkg, cuda, golden_dir):
    """tests/test_reference.cpp:99-114, abs tolerance 1e-4."""
    z = np.load(golden_dir / "pytorch_matmul.npz")
    for name in ["matmul", "matmul_batched", "matmul_shared"]:
        got = run_matmul(pkg, cuda, z[f"{name}/a"], z[f"{name}/b"])
        assert np.max(np.abs(got - z[f"{name}/output"])) <= 1e-4


def test_known_answers(pkg, cuda, golden_dir):
    spec = json.loads((golden_dir / "known_answers.json").read_text())
    for case in spec["products"]:
        a = np.array(case["a"], dtype=np.float32).reshape(case["a_shape"])
        b = np.array(case["b"], dtype=np.float32).reshape(case["b_shape"])
        out = run_matmul(pkg, cuda, a, b)
        assert list(out.shape) == case["out_shape"]
        if "out" in case:
            assert out.reshape(-1).tolist() == [float(v) for v in case["out"]]
        for idx, val in case.get("out_at", {}).items():
            assert out.reshape(-1)[int(idx)] == float(val)
    import torch

    for case in spec["throws"]:
        with pytest.raises(ValueError):
            pkg.matmul(torch.ones(case["a_shape"], device=cuda), torch.ones(case["b_shape"], device=cuda))


def test_seeded_configs_against_recorded_reference_outputs(pkg, orc, cuda, golden_dir):
    """Inputs rebuilt from the reference's seeds; outputs compared with the samples the
    unmodified reference engine produced (tests/golden/reference_runs.npz)."""
    import make_golden

    z = np.load(golden_dir / "reference_runs.npz")
    meta = json.loads((golden_dir / "reference_runs.json").read_text())
    for name in make_golden.CONFIGS:
        a, b = make_golden.config_inputs(name, orc.Rng)
        got = run_matmul(pkg, cuda, a, b)
        sample = got.reshape(-1)[::meta[name]["sample_step"]]
        assert orc.scaled_error(sample, z[f"{name}/sample"]) <= orc.parity_tolerance(a.shape[-1]), name


def test_edge_shapes(pkg, orc, cuda):
    import torch

    # empty products: nothing to compute, shapes still right (K == 0 gives zeros)
    assert pkg.matmul(torch.empty((0, 5), device=cuda), torch.empty((5, 3), device=cuda)).shape == (0, 3)
    out = pkg.matmul(torch.empty((4, 0), device=cuda), torch.empty((0, 3), device=cuda))
    pkg.status()
    assert out.shape == (4, 3) and not out.cpu().numpy().any()
    # exact zeros in A (the reference skips them) and signed zeros
    g = orc.Rng(16)
    a = np.maximum(g.randn((100, 64)), 0.0).astype(np.float32)
    b = g.randn((64, 33))
    assert orc.scaled_error(run_matmul(pkg, cuda, a, b), orc.matmul(a, b)) <= 1e-5
    # invalid arguments are refused before anything is launched
    with pytest.raises(pkg.B200Error):
        pkg.gemm(dev(a, cuda), dev(b, cuda), torch.empty((100, 33), device=cuda), batch=1, M=100, N=33, K=64,
                 lda=10, ldb=33, ldc=33)
    with pytest.raises(pkg.B200Error):
        pkg.gemm(dev(a, cuda), dev(b, cuda), None, batch=1, M=100, N=33, K=64, lda=64, ldb=33, ldc=33)
    with pytest.raises(pkg.B200Error):
        pkg.gemm(dev(a, cuda), dev(b, cuda), torch.empty((100, 33), device=cuda), batch=1, M=100, N=33, K=64,
                 lda=64, ldb=33, ldc=33, precision=7)


def test_tf32_mode_is_separate_and_less_precise(pkg, orc, cuda):
    """Plain TF32 is opt-in, bounded by the reference's 4*sqrt(K)*2^-11, and measurably worse
    than the default (tests/test_cuda_parity.cpp:392-419, 480-505)."""
    import torch

    g = orc.Rng(17)
    M = K = N = 256
    a, b = g.randn((M, K)), g.randn((K, N))
    want = orc.matmul_f64(a, b)
    A, B = dev(a, cuda), dev(b, cuda)
    C3 = torch.empty((M, N), device=cuda)
    C1 = torch.empty((M, N), device=cuda)
    gemm(pkg, cuda, A, B, C3, batch=1, M=M, N=N, K=K, lda=K, ldb=N, ldc=N)
    gemm(pkg, cuda, A, B, C1, batch=1, M=M, N=N, K=K, lda=K, ldb=N, ldc=N, precision=pkg.PRECISION_TF32)
    e3 = orc.scaled_error(C3.cpu().numpy(), want)
    e1 = orc.scaled_error(C1.cpu().numpy(), want)
    assert e1 <= 4.0 * np.sqrt(K) * 2.0 ** -11
    assert e3 <= 1e-5
    assert e1 > 10.0 * e3
    ai = np.random.default_rng(1).integers(-4, 5, size=(M, K)).astype(np.float32)
    bi = np.random.default_rng(2).integers(-4, 5, size=(K, N)).astype(np.float32)
    gemm(pkg, cuda, dev(ai, cuda), dev(bi, cuda), C1, batch=1, M=M, N=N, K=K, lda=K, ldb=N, ldc=N,
         precision=pkg.PRECISION_TF32)
    assert np.array_equal(C1.cpu().numpy(), orc.matmul(ai, bi))


def test_host_buffer_entry_point(pkg, orc, cuda):
    g = orc.Rng(18)
    a, b = g.randn((3, 50, 40)), g.randn((40, 30))
    out = np.full((3, 50, 30), np.nan, np.float32)
    pkg.matmul_host(a, b, out, batch=3, rows=50, inner=40, cols=30, a_batched=True, b_batched=False)
    assert orc.scaled_error(out, orc.matmul(a, b)) <= 1e-5


@pytest.mark.parametrize("M,K,N", [(4352, 640, 4608), (4096, 512, 9472)])
def test_host_buffer_entry_point_pipelined(pkg, orc, cuda, M, K, N):
    """Large products from host buffers run as a wavefront of row and column strips that overlaps
    uploads, kernels and downloads: every element of the result must still be the plain product
    (sampled rows against the CPU loop, every column; all of it finite and written), with panel
    counts that differ between rows and columns and panels that do not divide the matrix."""
    rng = np.random.default_rng(20)
    a = rng.standard_normal((M, K), dtype=np.float32)
    b = rng.standard_normal((K, N), dtype=np.float32)
    out = np.full((M, N), np.nan, np.float32)
    pkg.matmul_host(a, b, out, batch=1, rows=M, inner=K, cols=N, a_batched=False, b_batched=False)
    assert np.isfinite(out).all(), "a block of the result was never written"
    rows = np.unique(np.concatenate([np.arange(0, M, 173), [M - 1, 1023, 1024, 1535, 1536, 2047, 2048]]))
    want = orc.matmul(np.ascontiguousarray(a[rows]), b)
    assert orc.scaled_error(out[rows], want) <= orc.parity_tolerance(K)
    for panels in (3, 16, 0):  # other panel counts, and no pipelining at all: the same bits
        pkg.set_option("host_pipeline", panels)
        try:
            again = np.full((M, N), np.nan, np.float32)
            pkg.matmul_host(a, b, again, batch=1, rows=M, inner=K, cols=N, a_batched=False, b_batched=False)
        finally:
            pkg.set_option("host_pipeline", 1)
        assert orc.scaled_error(again, out) <= orc.parity_tolerance(K)


def test_long_contraction_over_few_tiles_is_split(pkg, orc, cuda):
    """512 x 512 x 8192: eight wide tiles would leave most of the GPU idle over a long k-loop, so
    the planner picks wide tiles AND splits K over the SMs (two launches).  Exact on integers,
    deterministic, within the K-dependent bound of the CPU loop on random inputs."""
    import torch

    M, N, K = 512, 512, 8192
    ws_bytes = pkg.workspace_bytes(1, M, N, K)
    assert ws_bytes >= 2 * M * N * 4, "expected a split-K plan for this shape"
    rng = np.random.default_rng(8)
    a = rng.integers(-4, 5, size=(M, K)).astype(np.float32)
    b = rng.integers(-3, 4, size=(K, N)).astype(np.float32)
    want = orc.matmul(a, b)
    A, B = dev(a, cuda), dev(b, cuda)
    outs = []
    before = pkg.launch_count()
    for _ in range(2):
        C = torch.empty((M, N), device=cuda)
        gemm(pkg, cuda, A, B, C, batch=1, M=M, N=N, K=K, lda=K, ldb=N, ldc=N, ws_bytes=ws_bytes)
        outs.append(C.cpu().numpy())
    assert pkg.launch_count() - before == 4, "product and reduction, twice"
    assert np.array_equal(outs[0], want) and np.array_equal(outs[0], outs[1])
    g = orc.Rng(9)
    ar, br = g.randn((M, K)), g.randn((K, N))
    C = torch.empty((M, N), device=cuda)
    gemm(pkg, cuda, dev(ar, cuda), dev(br, cuda), C, batch=1, M=M, N=N, K=K, lda=K, ldb=N, ldc=N, ws_bytes=ws_bytes)
    assert orc.scaled_error(C.cpu().numpy(), orc.matmul(ar, br)) <= orc.parity_tolerance(K)
