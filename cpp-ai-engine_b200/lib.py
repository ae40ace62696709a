"""ctypes binding of ``libb200gemm.so`` (the C ABI in ``include/b200_gemm.h``).

Arguments that are device buffers may be torch CUDA tensors (their ``data_ptr()`` is passed)
or plain integers holding a device address.  Nothing here computes: every function forwards
to the library and raises :class:`B200Error` on a non-zero return.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path
from typing import Optional, Sequence

from .build import LIB

PRECISION_3XTF32 = 0
PRECISION_TF32 = 1

_lib: Optional[ctypes.CDLL] = None

EXPORTS = (
    "b200_gemm_f32",
    "b200_attention_f32",
    "b200_attention_f32_strided",
    "b200_attention_backward_f32",
    "b200_attention_backward_f32_strided",
    "b200_conv2d_forward_f32",
    "b200_conv2d_backward_workspace",
    "b200_conv2d_backward_f32",
    "b200_gemm_f32_fused",
    "b200_gemm_f32_workspace",
    "b200_matmul_f32",
    "b200_matmul_f32_host",
    "b200_gemm_f32_colshard",
    "b200_gemm_f32_static_scratch",
    "b200_gemm_status",
    "b200_gemm_launch_count",
    "b200_gemm_set_option",
    "b200_gemm_strerror",
)


class Epilogue(ctypes.Structure):
    """``b200_epilogue``: bias[N], addend[M x N] (shared across the batch), relu flag."""
    _fields_ = [("bias", ctypes.c_void_p), ("addend", ctypes.c_void_p), ("ld_addend", ctypes.c_int64),
                ("relu", ctypes.c_int)]


class B200Error(RuntimeError):
    def __init__(self, code: int, where: str):
        self.code = code
        msg = load().b200_gemm_strerror(code)
        super().__init__(f"{where}: error {code}: {msg.decode() if msg else '?'}")


def lib_path() -> Path:
    return LIB


def load() -> ctypes.CDLL:
    """Loads the library; raises if it has not been built (no fallback exists)."""
    global _lib
    if _lib is not None:
        return _lib
    path = Path(os.environ.get("B200_GEMM_LIBRARY", str(LIB)))  # override: an alternative build
    if not path.exists():
        raise RuntimeError(
            f"{path} is missing: build it first (python -c 'import __graft_entry__ as g; g.build()')")
    lib = ctypes.CDLL(str(path))
    c_i64, c_f, c_vp, c_sz, c_int = ctypes.c_int64, ctypes.c_float, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
    lib.b200_gemm_f32.restype = c_int
    lib.b200_gemm_f32.argtypes = [c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_i64, c_int, c_int,
                                  c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_f, c_f, c_int,
                                  c_vp, c_sz, c_vp]
    lib.b200_gemm_f32_fused.restype = c_int
    lib.b200_gemm_f32_fused.argtypes = [c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_i64, c_int, c_int,
                                        c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_f, c_f, c_int,
                                        ctypes.POINTER(Epilogue), c_vp, c_sz, c_vp]
    lib.b200_attention_f32.restype = c_int
    lib.b200_attention_f32.argtypes = [c_vp] * 6 + [c_i64] * 5 + [c_f, c_int, c_vp]
    lib.b200_attention_f32_strided.restype = c_int
    lib.b200_attention_f32_strided.argtypes = ([c_vp] * 6 + [c_i64] * 6 + [ctypes.POINTER(c_i64)] * 4
                                               + [c_f, c_int, c_vp])
    lib.b200_attention_backward_f32.restype = c_int
    lib.b200_attention_backward_f32.argtypes = [c_vp] * 8 + [c_i64] * 5 + [c_f, c_f, c_int, c_vp]
    lib.b200_attention_backward_f32_strided.restype = c_int
    lib.b200_attention_backward_f32_strided.argtypes = ([c_vp] * 8 + [c_i64] * 6 + [ctypes.POINTER(c_i64)] * 4
                                                        + [c_f, c_f, c_int, c_vp])
    lib.b200_conv2d_forward_f32.restype = c_int
    lib.b200_conv2d_forward_f32.argtypes = [c_vp, c_vp, c_vp, c_vp] + [c_i64] * 9 + [c_int, c_int, c_vp]
    lib.b200_conv2d_backward_workspace.restype = c_sz
    lib.b200_conv2d_backward_workspace.argtypes = [c_i64] * 9
    lib.b200_conv2d_backward_f32.restype = c_int
    lib.b200_conv2d_backward_f32.argtypes = [c_vp] * 6 + [c_i64] * 9 + [c_f, c_int, c_vp, c_sz, c_vp]
    lib.b200_gemm_f32_workspace.restype = c_sz
    lib.b200_gemm_f32_workspace.argtypes = [c_i64, c_i64, c_i64, c_i64]
    lib.b200_matmul_f32.restype = c_int
    lib.b200_matmul_f32.argtypes = [c_vp, c_vp, c_vp, c_sz, c_sz, c_sz, c_sz, c_int, c_int, c_f,
                                    c_vp, c_sz, c_vp]
    lib.b200_matmul_f32_host.restype = c_int
    lib.b200_matmul_f32_host.argtypes = [c_vp, c_vp, c_vp, c_sz, c_sz, c_sz, c_sz, c_int, c_int, c_f]
    lib.b200_gemm_f32_colshard.restype = c_int
    lib.b200_gemm_f32_colshard.argtypes = [c_vp, c_vp, ctypes.POINTER(c_vp), c_int, c_i64, c_i64,
                                           c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_int, c_vp]
    lib.b200_gemm_f32_static_scratch.restype = c_int
    lib.b200_gemm_f32_static_scratch.argtypes = [c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_i64, c_int, c_int,
                                                 c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_f, c_f,
                                                 c_int, c_vp, c_vp]
    lib.b200_gemm_status.restype = c_int
    lib.b200_gemm_status.argtypes = []
    lib.b200_gemm_launch_count.restype = ctypes.c_uint64
    lib.b200_gemm_launch_count.argtypes = []
    lib.b200_gemm_set_option.restype = c_int
    lib.b200_gemm_set_option.argtypes = [ctypes.c_char_p, ctypes.c_long]
    lib.b200_gemm_strerror.restype = ctypes.c_char_p
    lib.b200_gemm_strerror.argtypes = [c_int]
    _lib = lib
    return lib


def _ptr(x) -> int:
    if x is None:
        return 0
    if isinstance(x, int):
        return x
    return int(x.data_ptr())


def _stream_ptr(stream) -> int:
    if stream is None:
        import torch

        return int(torch.cuda.current_stream().cuda_stream)
    if isinstance(stream, int):
        return stream
    return int(stream.cuda_stream)


def _check(rc: int, where: str) -> None:
    if rc != 0:
        raise B200Error(rc, where)


def gemm(A, B, C, *, batch: int, M: int, N: int, K: int, transA: bool = False, transB: bool = False,
         lda: int, ldb: int, ldc: int, strideA: int = 0, strideB: int = 0, strideC: int = 0,
         alpha: float = 1.0, beta: float = 0.0, precision: int = PRECISION_3XTF32,
         workspace=None, workspace_bytes: int = 0, stream=None) -> None:
    """``C[b] = alpha * op(A[b]) @ op(B[b]) + beta * C[b]`` — forwards to ``b200_gemm_f32``."""
    rc = load().b200_gemm_f32(_ptr(A), _ptr(B), _ptr(C), batch, M, N, K, int(transA), int(transB),
                              lda, ldb, ldc, strideA, strideB, strideC, alpha, beta, precision,
                              _ptr(workspace), workspace_bytes, _stream_ptr(stream))
    _check(rc, "b200_gemm_f32")


def gemm_static_scratch(A, B, C, *, batch: int, M: int, N: int, K: int, transA: bool = False,
                        transB: bool = False, lda: int, ldb: int, ldc: int, strideA: int = 0,
                        strideB: int = 0, strideC: int = 0, alpha: float = 1.0, beta: float = 0.0,
                        precision: int = PRECISION_3XTF32, device_status=None, stream=None) -> None:
    """Same product as :func:`gemm` through ``b200_gemm_f32_static_scratch``: the split-K scratch
    is the fixed array inside the library, nothing is allocated.  ``device_status`` is an optional
    int32 CUDA tensor (zeroed by the caller) that receives device-side timeout bits."""
    rc = load().b200_gemm_f32_static_scratch(_ptr(A), _ptr(B), _ptr(C), batch, M, N, K, int(transA),
                                             int(transB), lda, ldb, ldc, strideA, strideB, strideC,
                                             alpha, beta, precision, _ptr(device_status),
                                             _stream_ptr(stream))
    _check(rc, "b200_gemm_f32_static_scratch")


def gemm_fused(A, B, C, *, batch: int, M: int, N: int, K: int, transA: bool = False, transB: bool = False,
               lda: int, ldb: int, ldc: int, strideA: int = 0, strideB: int = 0, strideC: int = 0,
               alpha: float = 1.0, beta: float = 0.0, precision: int = PRECISION_3XTF32, bias=None,
               addend=None, ld_addend: int = 0, relu: bool = False, workspace=None, workspace_bytes: int = 0,
               stream=None) -> None:
    """``C = relu?(alpha * op(A) @ op(B) + bias[col] + addend[row, col] + beta * C)`` in one kernel."""
    ep = Epilogue(_ptr(bias) or None, _ptr(addend) or None, ld_addend or N, int(relu))
    rc = load().b200_gemm_f32_fused(_ptr(A), _ptr(B), _ptr(C), batch, M, N, K, int(transA), int(transB),
                                    lda, ldb, ldc, strideA, strideB, strideC, alpha, beta, precision,
                                    ctypes.byref(ep), _ptr(workspace), workspace_bytes, _stream_ptr(stream))
    _check(rc, "b200_gemm_f32_fused")


def attention_forward(q, k, v, mask, out, weights, *, batch: int, s_q: int, s_k: int, d_k: int, d_v: int,
                      scale: float, precision: int = PRECISION_3XTF32, stream=None) -> None:
    """``out = softmax(q @ k^T * scale + mask) @ v`` per batch element, one fused kernel."""
    rc = load().b200_attention_f32(_ptr(q), _ptr(k), _ptr(v), _ptr(mask), _ptr(out), _ptr(weights), batch, s_q,
                                   s_k, d_k, d_v, scale, precision, _stream_ptr(stream))
    _check(rc, "b200_attention_f32")


def attention_forward_strided(q, k, v, mask, out, weights, *, batch: int, heads: int, s_q: int, s_k: int, d_k: int,
                              d_v: int, q_strides, k_strides, v_strides, out_strides, scale: float,
                              precision: int = PRECISION_3XTF32, stream=None) -> None:
    """The fused attention kernel over ``batch * heads`` matrices addressed by (batch, head, row) strides in
    floats: the split into heads and the merge back cost no copy."""
    arr = ctypes.c_int64 * 3
    rc = load().b200_attention_f32_strided(_ptr(q), _ptr(k), _ptr(v), _ptr(mask), _ptr(out), _ptr(weights), batch,
                                           heads, s_q, s_k, d_k, d_v, arr(*q_strides), arr(*k_strides),
                                           arr(*v_strides), arr(*out_strides), scale, precision,
                                           _stream_ptr(stream))
    _check(rc, "b200_attention_f32_strided")


def attention_backward_strided(q, k, v, mask, dout, dq, dk, dv, *, batch: int, heads: int, s_q: int, s_k: int,
                               d_k: int, d_v: int, q_strides, k_strides, v_strides, out_strides, scale: float,
                               beta: float = 0.0, precision: int = PRECISION_3XTF32, stream=None) -> None:
    """Gradients of the fused attention core (dq, dk, dv addressed like q, k, v; dout like out), one kernel."""
    arr = ctypes.c_int64 * 3
    rc = load().b200_attention_backward_f32_strided(
        _ptr(q), _ptr(k), _ptr(v), _ptr(mask), _ptr(dout), _ptr(dq), _ptr(dk), _ptr(dv), batch, heads, s_q, s_k, d_k,
        d_v, arr(*q_strides), arr(*k_strides), arr(*v_strides), arr(*out_strides), scale, beta, precision,
        _stream_ptr(stream))
    _check(rc, "b200_attention_backward_f32_strided")


def conv2d_backward_workspace(*, n: int, c: int, h: int, w: int, out_c: int, kh: int, kw: int, stride: int = 1,
                              pad: int = 0) -> int:
    """Bytes of workspace the weight gradient of this convolution wants."""
    return int(load().b200_conv2d_backward_workspace(n, c, h, w, out_c, kh, kw, stride, pad))


def conv2d_backward(x, weight, dy, dx, dweight, dbias, *, n: int, c: int, h: int, w: int, out_c: int, kh: int,
                    kw: int, stride: int = 1, pad: int = 0, beta: float = 0.0, precision: int = PRECISION_3XTF32,
                    workspace=None, workspace_bytes: int = 0, stream=None) -> None:
    """Gradients of ``conv2d`` (each of dx, dweight, dbias optional): implicit-GEMM kernels, no column matrix."""
    rc = load().b200_conv2d_backward_f32(_ptr(x), _ptr(weight), _ptr(dy), _ptr(dx), _ptr(dweight), _ptr(dbias), n, c,
                                         h, w, out_c, kh, kw, stride, pad, beta, precision, _ptr(workspace),
                                         workspace_bytes, _stream_ptr(stream))
    _check(rc, "b200_conv2d_backward_f32")


def conv2d_forward(x, weight, bias, y, *, n: int, c: int, h: int, w: int, out_c: int, kh: int, kw: int,
                   stride: int = 1, pad: int = 0, relu: bool = False, precision: int = PRECISION_3XTF32,
                   stream=None) -> None:
    """``y = conv2d(x, weight) + bias`` (NCHW) as one implicit-GEMM kernel."""
    rc = load().b200_conv2d_forward_f32(_ptr(x), _ptr(weight), _ptr(bias), _ptr(y), n, c, h, w, out_c, kh, kw,
                                        stride, pad, int(relu), precision, _stream_ptr(stream))
    _check(rc, "b200_conv2d_forward_f32")


def workspace_bytes(batch: int, M: int, N: int, K: int) -> int:
    return int(load().b200_gemm_f32_workspace(batch, M, N, K))


def matmul_host(a, b, out, *, batch: int, rows: int, inner: int, cols: int, a_batched: bool,
                b_batched: bool, beta: float = 0.0) -> None:
    """Host-buffer product (numpy float32 arrays): upload, kernel, download, synchronised."""
    rc = load().b200_matmul_f32_host(a.ctypes.data, b.ctypes.data, out.ctypes.data, batch, rows,
                                     inner, cols, int(a_batched), int(b_batched), beta)
    _check(rc, "b200_matmul_f32_host")


def gemm_colshard(A, B, dest: Sequence, *, M: int, N: int, K: int, col0: int, cols: int,
                  lda: int, ldb: int, ldc: int, precision: int = PRECISION_3XTF32, stream=None) -> None:
    """Columns ``[col0, col0+cols)`` of ``A @ B`` stored into every buffer of ``dest``."""
    arr = (ctypes.c_void_p * len(dest))(*[_ptr(d) for d in dest])
    rc = load().b200_gemm_f32_colshard(_ptr(A), _ptr(B), arr, len(dest), M, N, K, col0, cols, lda,
                                       ldb, ldc, precision, _stream_ptr(stream))
    _check(rc, "b200_gemm_f32_colshard")


def status() -> None:
    """Synchronises the current device and raises if a bounded device-side wait ran out."""
    _check(load().b200_gemm_status(), "b200_gemm_status")


def launch_count() -> int:
    return int(load().b200_gemm_launch_count())


def set_option(name: str, value: int) -> None:
    _check(load().b200_gemm_set_option(name.encode(), int(value)), f"b200_gemm_set_option({name})")
