"""Generates the golden vectors under tests/golden/ (run in the build container, where the
reference tree and the reference CPU build oracle/_ref are present):

    python tests/golden/make_golden.py [--reference <reference source tree>]

Outputs (small, committed):
  pytorch_matmul.npz / .bin   the reference's own PyTorch golden vectors for its matrix product and
                       its gradients (tests/fixtures/matmul*.bin, consumed by
                       tests/test_reference.cpp:99-114), re-encoded as npz.
  pytorch_conv2d.npz   the reference's PyTorch golden vectors for Conv2d forward and backward
                       (tests/fixtures/conv2d_*.bin).
  reference_conv_backward.npz  the UNMODIFIED reference engine's Conv2d forward + autograd backward on
                       seeded inputs (drawn from its own generator): inputs, output and the three gradients.
  pytorch_attention.npz  the reference's PyTorch golden vectors for attention forward and backward
                       (tests/fixtures/attention*.bin).
  reference_attention_backward.npz  the UNMODIFIED reference engine's scaled_dot_product_attention + autograd on
                       seeded inputs: output and the three gradients (the inputs are re-drawn from the seed).
  pytorch_multihead.npz  the same for a whole MultiHeadAttention forward (tests/fixtures/multihead_attention.bin).
  pytorch_layers.bin   the Conv2d, attention and MultiHeadAttention vectors again, in the container format,
                       for the C++ host tests.
  known_answers.json   the integer known-answer products of tests/test_tensor.cpp:47-65, 182-202.
  reference_runs.npz   outputs of the UNMODIFIED reference engine (oracle/_ref) on seeded
                       inputs: its random streams, and per configuration a SHA-256 of the full
                       product plus a strided sample of it.

The fixture container format read here is the reference's documented one
(include/engine/serialize.hpp:12-31): "CPPAIENG", u32 version, u32 count, then per tensor
u32 name length, name, u32 ndim, u64 dims, f32 data; little-endian.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import struct
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))

from oracle import oracle_py as orc  # noqa: E402


def read_fixture(path: Path) -> dict:
    raw = path.read_bytes()
    if raw[:8] != b"CPPAIENG":
        raise ValueError(f"{path}: bad signature")
    version, count = struct.unpack_from("<II", raw, 8)
    if version != 1:
        raise ValueError(f"{path}: version {version}")
    off = 16
    out = {}
    for _ in range(count):
        (nlen,) = struct.unpack_from("<I", raw, off)
        off += 4
        name = raw[off:off + nlen].decode()
        off += nlen
        (ndim,) = struct.unpack_from("<I", raw, off)
        off += 4
        dims = struct.unpack_from(f"<{ndim}Q", raw, off)
        off += 8 * ndim
        n = int(np.prod(dims)) if ndim else 1
        out[name] = np.frombuffer(raw, dtype="<f4", count=n, offset=off).reshape(dims).copy()
        off += 4 * n
    return out


def write_container(path: Path, tensors: dict) -> None:
    """Writes tensors in the same documented container format (version 1, little-endian)."""
    out = bytearray(b"CPPAIENG")
    out += struct.pack("<II", 1, len(tensors))
    for name, val in tensors.items():
        val = np.ascontiguousarray(val, dtype="<f4")
        raw_name = name.encode()
        out += struct.pack("<I", len(raw_name)) + raw_name
        out += struct.pack("<I", val.ndim) + struct.pack(f"<{val.ndim}Q", *val.shape)
        out += val.tobytes()
    path.write_bytes(bytes(out))


def sha(x: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(x, dtype="<f4").tobytes()).hexdigest()


# The seeded configurations the parity tests use, built exactly like a program using the
# reference would build them: manual_seed, then tensors drawn in this order.
def config_inputs(name: str, rng_factory):
    if name == "cfg1_512":  # bench_matmul-shaped product, U[-1,1], seed 0
        g = rng_factory(0)
        return g.rand((512, 512), -1.0, 1.0), g.rand((512, 512), -1.0, 1.0)
    if name == "det_200x150x120":  # tests/test_tensor.cpp:456-476
        g = rng_factory(7)
        return g.randn((200, 150)), g.randn((150, 120))
    if name == "cfg4_relu_256":  # half-zero A, reduced size of the relu-sparse case, seed 4
        g = rng_factory(4)
        a = np.maximum(g.randn((256, 256)), 0.0).astype(np.float32)
        return a, g.randn((256, 256))
    if name == "cfg2_scores":  # batched per-head Q x K^T operands (K^T materialised), seed 2
        g = rng_factory(2)
        q = g.randn((8, 64, 24))
        k = g.randn((8, 64, 24))
        return q, np.ascontiguousarray(np.swapaxes(k, 1, 2))
    if name == "cfg2_shared":  # (B, M, K) x (K, N): Linear on a batch, Xavier-uniform weight
        g = rng_factory(2)
        x = g.randn((4, 64, 96))
        bound = float(np.sqrt(6.0 / (96 + 121)))
        return x, g.rand((96, 121), -bound, bound)
    raise KeyError(name)


# (lead, s_q, s_k, d_k, d_v, causal) of the recorded attention-backward runs, inputs from seed 13
ATTENTION_BACKWARD_CASES = {"charlm_heads": (2, 64, 64, 24, 24, True), "ragged": (3, 17, 33, 9, 20, False)}


def attention_backward_inputs(tag: str, rng_factory):
    lead, s_q, s_k, d_k, d_v, causal = ATTENTION_BACKWARD_CASES[tag]
    g = rng_factory(13)
    q, k, v = g.randn((lead, s_q, d_k)), g.randn((lead, s_k, d_k)), g.randn((lead, s_k, d_v))
    go = g.randn((lead, s_q, d_v))
    mask = np.triu(np.full((s_q, s_k), -1e9, np.float32), 1) if causal else None
    return q, k, v, go, mask


CONFIGS = ["cfg1_512", "det_200x150x120", "cfg4_relu_256", "cfg2_scores", "cfg2_shared"]


class RefRng:
    """The reference engine's own global generator."""

    def __init__(self, seed: int):
        import ctypes

        orc.ref().ref_manual_seed(ctypes.c_uint64(seed))

    def rand(self, shape, lo=-1.0, hi=1.0):
        import ctypes

        out = np.empty(shape, dtype=np.float32)
        orc.ref().ref_rand(out.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), ctypes.c_size_t(out.size),
                           ctypes.c_float(lo), ctypes.c_float(hi))
        return out

    def randn(self, shape, mean=0.0, stddev=1.0):
        import ctypes

        out = np.empty(shape, dtype=np.float32)
        orc.ref().ref_randn(out.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), ctypes.c_size_t(out.size),
                            ctypes.c_float(mean), ctypes.c_float(stddev))
        return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default="/root/reference")
    args = ap.parse_args()
    ref_dir = Path(args.reference)

    # 1. the reference's PyTorch golden vectors
    packed = {}
    for name in ["matmul", "matmul_batched", "matmul_shared"]:
        fx = read_fixture(ref_dir / "tests" / "fixtures" / f"{name}.bin")
        for key, val in fx.items():
            packed[f"{name}/{key}"] = val
    np.savez(HERE / "pytorch_matmul.npz", **packed)
    write_container(HERE / "pytorch_matmul.bin", packed)  # same vectors for the C++ host tests

    # 1b. the reference's PyTorch golden vectors for Conv2d (tests/fixtures/conv2d_*.bin,
    #     consumed by tests/test_reference.cpp:216-251): inputs, parameters and outputs
    conv = {}
    for name in ["conv2d_pad1", "conv2d_stride2"]:
        fx = read_fixture(ref_dir / "tests" / "fixtures" / f"{name}.bin")
        for key in ("input", "weight", "bias", "output", "grad_output", "grad.input", "grad.weight", "grad.bias"):
            conv[f"{name}/{key}"] = fx[key]
    np.savez(HERE / "pytorch_conv2d.npz", **conv)

    # 1c. the reference's PyTorch golden vectors for scaled dot-product attention
    #     (tests/fixtures/attention*.bin, consumed by tests/test_reference.cpp:296-340)
    att = {}
    for name in ["attention", "attention_causal"]:
        fx = read_fixture(ref_dir / "tests" / "fixtures" / f"{name}.bin")
        for key, val in fx.items():
            att[f"{name}/{key}"] = val
    np.savez(HERE / "pytorch_attention.npz", **att)

    # 1c'. the reference engine's own attention + autograd on seeded inputs.  Only the results are
    #      stored: the inputs are drawn again from the same seed by attention_backward_inputs()
    #      (the oracle's generator reproduces the reference's streams bit for bit, see section 3).
    ab = {}
    for tag in ATTENTION_BACKWARD_CASES:
        q, k, v, go, mask = attention_backward_inputs(tag, RefRng)
        out, w, gq, gk, gv = orc.ref_attention_backward(q, k, v, mask, go)
        for key, val in (("output", out), ("grad.q", gq), ("grad.k", gk), ("grad.v", gv)):
            ab[f"{tag}/{key}"] = val
    np.savez(HERE / "reference_attention_backward.npz", **ab)

    # 1d. the reference's PyTorch golden vectors for MultiHeadAttention(8, 2) forward
    #     (tests/fixtures/multihead_attention.bin, consumed by tests/test_reference.cpp:322-349):
    #     input, the four projections' weights (in, out) and biases, output
    fx = read_fixture(ref_dir / "tests" / "fixtures" / "multihead_attention.bin")
    np.savez(HERE / "pytorch_multihead.npz", **{k: v for k, v in fx.items() if not k.startswith("grad")})

    # 1d'. the same layer vectors (Conv2d with gradients, attention, MultiHeadAttention) in the container
    #      format, for the C++ host tests
    layers = dict(conv)
    layers.update(att)
    layers.update({f"multihead/{k}": v for k, v in fx.items() if not k.startswith("grad")})
    write_container(HERE / "pytorch_layers.bin", layers)

    # 1e. the reference engine's own Conv2d layer and autograd on seeded inputs
    cb = {}
    for tag, (n, c, h, w, oc, k, stride, pad) in {"pad1": (2, 3, 9, 7, 5, 3, 1, 1), "stride2": (3, 2, 11, 8, 4, 3, 2, 0),
                                                  "k5pad2": (1, 4, 6, 6, 3, 5, 1, 2)}.items():
        g = RefRng(11)
        x, wt, b = g.randn((n, c, h, w)), g.rand((oc, c, k, k), -0.5, 0.5), g.rand((oc,), -0.5, 0.5)
        oh, ow = (h + 2 * pad - k) // stride + 1, (w + 2 * pad - k) // stride + 1
        dy = g.randn((n, oc, oh, ow))
        y, gx, gw, gb = orc.ref_conv2d_backward(x, wt, b, dy, stride, pad)
        for key, val in (("x", x), ("weight", wt), ("bias", b), ("grad_output", dy), ("output", y), ("grad.x", gx),
                         ("grad.weight", gw), ("grad.bias", gb)):
            cb[f"{tag}/{key}"] = val
        cb[f"{tag}/window"] = np.array([stride, pad], np.int64)
    np.savez(HERE / "reference_conv_backward.npz", **cb)

    # 2. integer known answers (tests/test_tensor.cpp:47-65, 182-202)
    known = [
        {"a_shape": [2, 3], "a": [1, 2, 3, 4, 5, 6], "b_shape": [3, 2], "b": [7, 8, 9, 1, 2, 3],
         "out_shape": [2, 2], "out": [31, 19, 85, 55]},
        {"a_shape": [2, 2, 3], "a": list(range(1, 13)), "b_shape": [2, 3, 2],
         "b": [1, 0, 0, 1, 1, 1, 2, 0, 0, 2, 1, 1], "out_shape": [2, 2, 2],
         "out_at": {"0": 4, "1": 5, "4": 23}},
        {"a_shape": [2, 2, 3], "a": list(range(1, 13)), "b_shape": [3, 2], "b": [1, 0, 0, 1, 1, 1],
         "out_shape": [2, 2, 2], "out_at": {"0": 4, "4": 16}},
    ]
    throws = [
        {"a_shape": [2, 3], "b_shape": [2, 3], "why": "incompatible inner dimensions"},
        {"a_shape": [2, 2, 3], "b_shape": [3, 3, 2], "why": "mismatched batches"},
        {"a_shape": [4], "b_shape": [4], "why": "1-D operands"},
    ]
    (HERE / "known_answers.json").write_text(json.dumps({"products": known, "throws": throws}, indent=1))

    # 3. outputs of the unmodified reference engine
    runs = {}
    for seed in (0, 1, 7):
        g = RefRng(seed)
        runs[f"rng/seed{seed}/rand"] = g.rand((33,), -1.0, 1.0)
        runs[f"rng/seed{seed}/randn"] = g.randn((33,), 0.5, 2.0)
        runs[f"rng/seed{seed}/rand_after"] = g.rand((4,), 0.0, 1.0)
    meta = {}
    for name in CONFIGS:
        a, b = config_inputs(name, RefRng)
        c = orc.ref_matmul(a, b)
        flat = c.reshape(-1)
        step = max(1, flat.size // 509)
        runs[f"{name}/sample"] = flat[::step].copy()
        meta[name] = {"a_sha256": sha(a), "b_sha256": sha(b), "out_sha256": sha(c), "sample_step": step,
                      "out_shape": list(c.shape)}
        # gradients through the reference's autograd for an explicit grad_output
        import ctypes

        gseed = RefRng(99)
        gout = gseed.randn(c.shape)
        ga, gb = np.empty_like(a), np.empty_like(b)
        fp = ctypes.POINTER(ctypes.c_float)
        dims = c.shape[:-2]
        batch = int(np.prod(dims)) if dims else 1
        rc = orc.ref().ref_matmul_backward(
            a.ctypes.data_as(fp), b.ctypes.data_as(fp), gout.ctypes.data_as(fp), None,
            ga.ctypes.data_as(fp), gb.ctypes.data_as(fp), ctypes.c_size_t(batch),
            ctypes.c_size_t(a.shape[-2]), ctypes.c_size_t(a.shape[-1]), ctypes.c_size_t(b.shape[-1]),
            int(a.ndim > 2), int(b.ndim > 2))
        assert rc == 0
        meta[name]["grad_a_sha256"] = sha(ga)
        meta[name]["grad_b_sha256"] = sha(gb)
    np.savez(HERE / "reference_runs.npz", **runs)
    (HERE / "reference_runs.json").write_text(json.dumps(meta, indent=1))
    print("wrote", [p.name for p in sorted(HERE.glob("*.np*"))], "known_answers.json reference_runs.json")


if __name__ == "__main__":
    main()
