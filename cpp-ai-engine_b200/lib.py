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
    "b200_attention_any_workspace",
    "b200_attention_any_f32",
    "b200_attention_backward_any_f32",
    "b200_conv2d_forward_f32",
    "b200_conv2d_backward_workspace",
    "b200_conv2d_backward_f32",
    "b200_gemm_f32_fused",
    "b200_gemm_f32_workspace",
    "b200_gemm_f32_plan",
    "b200_matmul_f32",
    "b200_matmul_f32_host",
    "b200_gemm_f32_colshard",
    "b200_shard_comm_create",
    "b200_shard_comm_set_peers",
    "b200_shard_comm_set_nccl",
    "b200_shard_comm_destroy",
    "b200_shard_columns",
    "b200_gemm_f32_sharded",
    "b200_shard_host_plan",
    "b200_matmul_f32_host_sharded",
    "b200_gemm_f32_static_scratch",
    "b200_gemm_status",
    "b200_gemm_selftest_timeout",
    "b200_gemm_launch_count",
    "b200_gemm_set_option",
    "b200_gemm_strerror",
)


class Epilogue(ctypes.Structure):
    """``b200_epilogue``: bias[N], addend[M x N] (shared across the batch), relu flag."""
    _fields_ = [("bias", ctypes.c_void_p), ("addend", ctypes.c_void_p), ("ld_addend", ctypes.c_int64),
                ("relu", ctypes.c_int)]


class PlanInfo(ctypes.Structure):
    """``b200_plan_info``: what one call of ``b200_gemm_f32`` would launch."""
    _fields_ = [("tile_n", ctypes.c_int), ("pair", ctypes.c_int), ("split_k", ctypes.c_int),
                ("tail_tiles", ctypes.c_int), ("tail_split", ctypes.c_int), ("kernels", ctypes.c_int),
                ("workspace_used", ctypes.c_size_t)]


class ShardHostLayout(ctypes.Structure):
    """``b200_shard_host_layout``: how the rows of A are cut for the sharded host-buffer product."""
    _fields_ = [("chunks", ctypes.c_int), ("rows_per_rank", ctypes.c_int64), ("chunk_rows", ctypes.c_int64)]


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
    lib.b200_attention_any_workspace.restype = c_sz
    lib.b200_attention_any_workspace.argtypes = [c_i64] * 6 + [c_int]
    lib.b200_attention_any_f32.restype = c_int
    lib.b200_attention_any_f32.argtypes = ([c_vp] * 6 + [c_i64] * 6 + [ctypes.POINTER(c_i64)] * 4
                                           + [c_f, c_int, c_vp, c_sz, c_vp])
    lib.b200_attention_backward_any_f32.restype = c_int
    lib.b200_attention_backward_any_f32.argtypes = ([c_vp] * 8 + [c_i64] * 6 + [ctypes.POINTER(c_i64)] * 4
                                                    + [c_f, c_f, c_int, c_vp, c_sz, c_vp])
    lib.b200_conv2d_forward_f32.restype = c_int
    lib.b200_conv2d_forward_f32.argtypes = [c_vp, c_vp, c_vp, c_vp] + [c_i64] * 9 + [c_int, c_int, c_vp]
    lib.b200_conv2d_backward_workspace.restype = c_sz
    lib.b200_conv2d_backward_workspace.argtypes = [c_i64] * 9
    lib.b200_conv2d_backward_f32.restype = c_int
    lib.b200_conv2d_backward_f32.argtypes = [c_vp] * 6 + [c_i64] * 9 + [c_f, c_int, c_vp, c_sz, c_vp]
    lib.b200_gemm_f32_workspace.restype = c_sz
    lib.b200_gemm_f32_workspace.argtypes = [c_i64, c_i64, c_i64, c_i64]
    lib.b200_gemm_f32_plan.restype = c_int
    lib.b200_gemm_f32_plan.argtypes = [c_i64, c_i64, c_i64, c_i64, c_sz, ctypes.POINTER(PlanInfo)]
    lib.b200_matmul_f32.restype = c_int
    lib.b200_matmul_f32.argtypes = [c_vp, c_vp, c_vp, c_sz, c_sz, c_sz, c_sz, c_int, c_int, c_f,
                                    c_vp, c_sz, c_vp]
    lib.b200_matmul_f32_host.restype = c_int
    lib.b200_matmul_f32_host.argtypes = [c_vp, c_vp, c_vp, c_sz, c_sz, c_sz, c_sz, c_int, c_int, c_f]
    lib.b200_gemm_f32_colshard.restype = c_int
    lib.b200_gemm_f32_colshard.argtypes = [c_vp, c_vp, ctypes.POINTER(c_vp), c_int, c_i64, c_i64,
                                           c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_int, c_vp]
    lib.b200_shard_comm_create.restype = c_int
    lib.b200_shard_comm_create.argtypes = [ctypes.POINTER(c_vp), c_int, c_int]
    lib.b200_shard_comm_set_peers.restype = c_int
    lib.b200_shard_comm_set_peers.argtypes = [c_vp, ctypes.POINTER(c_vp), ctypes.POINTER(c_vp)]
    lib.b200_shard_comm_set_nccl.restype = c_int
    lib.b200_shard_comm_set_nccl.argtypes = [c_vp, c_vp]
    lib.b200_shard_comm_destroy.restype = c_int
    lib.b200_shard_comm_destroy.argtypes = [c_vp]
    lib.b200_shard_columns.restype = None
    lib.b200_shard_columns.argtypes = [c_i64, c_int, c_int, ctypes.POINTER(c_i64), ctypes.POINTER(c_i64)]
    lib.b200_gemm_f32_sharded.restype = c_int
    lib.b200_gemm_f32_sharded.argtypes = [c_vp, c_int, c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64,
                                          c_int, c_vp]
    lib.b200_shard_host_plan.restype = c_int
    lib.b200_shard_host_plan.argtypes = [c_i64, c_int, c_int, ctypes.POINTER(ShardHostLayout)]
    lib.b200_matmul_f32_host_sharded.restype = c_int
    lib.b200_matmul_f32_host_sharded.argtypes = [c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_int]
    lib.b200_gemm_f32_static_scratch.restype = c_int
    lib.b200_gemm_f32_static_scratch.argtypes = [c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_i64, c_int, c_int,
                                                 c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_f, c_f,
                                                 c_int, c_vp, c_vp]
    lib.b200_gemm_status.restype = c_int
    lib.b200_gemm_status.argtypes = []
    lib.b200_gemm_selftest_timeout.restype = c_int
    lib.b200_gemm_selftest_timeout.argtypes = [ctypes.c_uint, ctypes.POINTER(c_int)]
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

        # the raw handle of torch's current stream on the current device (no Stream object is built:
        # this runs once per product, and an engine-sized product is a few microseconds)
        return torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice())
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


def attention_any_workspace(*, batch: int, heads: int, s_q: int, s_k: int, d_k: int, d_v: int,
                            backward: bool = False) -> int:
    """Bytes of workspace ``attention_any`` / ``attention_backward_any`` want for this shape (0: fused kernel)."""
    return int(load().b200_attention_any_workspace(batch, heads, s_q, s_k, d_k, d_v, int(backward)))


def attention_any(q, k, v, mask, out, weights, *, batch: int, heads: int, s_q: int, s_k: int, d_k: int, d_v: int,
                  q_strides, k_strides, v_strides, out_strides, scale: float, precision: int = PRECISION_3XTF32,
                  workspace=None, workspace_bytes: int = 0, stream=None) -> None:
    """Attention for heads of any size: the fused kernel when the head fits it, else composed on the device."""
    arr = ctypes.c_int64 * 3
    rc = load().b200_attention_any_f32(_ptr(q), _ptr(k), _ptr(v), _ptr(mask), _ptr(out), _ptr(weights), batch, heads,
                                       s_q, s_k, d_k, d_v, arr(*q_strides), arr(*k_strides), arr(*v_strides),
                                       arr(*out_strides), scale, precision, _ptr(workspace), workspace_bytes,
                                       _stream_ptr(stream))
    _check(rc, "b200_attention_any_f32")


def attention_backward_any(q, k, v, mask, dout, dq, dk, dv, *, batch: int, heads: int, s_q: int, s_k: int, d_k: int,
                           d_v: int, q_strides, k_strides, v_strides, out_strides, scale: float, beta: float = 0.0,
                           precision: int = PRECISION_3XTF32, workspace=None, workspace_bytes: int = 0,
                           stream=None) -> None:
    """Gradients of :func:`attention_any`, any size."""
    arr = ctypes.c_int64 * 3
    rc = load().b200_attention_backward_any_f32(
        _ptr(q), _ptr(k), _ptr(v), _ptr(mask), _ptr(dout), _ptr(dq), _ptr(dk), _ptr(dv), batch, heads, s_q, s_k, d_k,
        d_v, arr(*q_strides), arr(*k_strides), arr(*v_strides), arr(*out_strides), scale, beta, precision,
        _ptr(workspace), workspace_bytes, _stream_ptr(stream))
    _check(rc, "b200_attention_backward_any_f32")


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


def plan(batch: int, M: int, N: int, K: int, workspace_bytes: int = 2 ** 62) -> dict:
    """The tile, K-split and kernel count ``gemm`` would use for this shape and workspace."""
    info = PlanInfo()
    _check(load().b200_gemm_f32_plan(batch, M, N, K, workspace_bytes, ctypes.byref(info)), "b200_gemm_f32_plan")
    return {name: int(getattr(info, name)) for name, _ in PlanInfo._fields_}


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


SHARD_FUSED = 0
SHARD_NCCL = 1


class ShardComm:
    """``b200_shard_comm``: the handle of the sharded products (one per rank, on the current device)."""

    def __init__(self, rank: int, world: int):
        self._h = ctypes.c_void_p()
        _check(load().b200_shard_comm_create(ctypes.byref(self._h), rank, world), "b200_shard_comm_create")
        self.rank, self.world = rank, world

    def set_peers(self, c_bufs: Sequence, flags: Sequence) -> None:
        """Every rank's C buffer and zeroed flag block (tensors or device addresses, index = rank)."""
        arr_c = (ctypes.c_void_p * self.world)(*[_ptr(t) for t in c_bufs])
        arr_f = (ctypes.c_void_p * self.world)(*[_ptr(t) for t in flags])
        _check(load().b200_shard_comm_set_peers(self._h, arr_c, arr_f), "b200_shard_comm_set_peers")

    def set_nccl(self, comm_ptr: int) -> None:
        """The caller's ``ncclComm_t`` of the same ranks, as an integer address."""
        _check(load().b200_shard_comm_set_nccl(self._h, ctypes.c_void_p(comm_ptr)), "b200_shard_comm_set_nccl")

    def close(self) -> None:
        if self._h:
            load().b200_shard_comm_destroy(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def shard_columns(N: int, world: int, rank: int):
    """``b200_shard_columns``: the (col0, cols) of a rank, as the library computes them."""
    c0, c = ctypes.c_int64(), ctypes.c_int64()
    load().b200_shard_columns(N, world, rank, ctypes.byref(c0), ctypes.byref(c))
    return int(c0.value), int(c.value)


def shard_host_plan(M: int, world: int, chunks: int = 0) -> dict:
    """``b200_shard_host_plan``: chunks, rows per rank and rows per chunk of the sharded host product."""
    lay = ShardHostLayout()
    _check(load().b200_shard_host_plan(M, world, chunks, ctypes.byref(lay)), "b200_shard_host_plan")
    return {"chunks": int(lay.chunks), "rows_per_rank": int(lay.rows_per_rank), "chunk_rows": int(lay.chunk_rows)}


def gemm_sharded(comm: ShardComm, mode: int, A, B, C, *, M: int, N: int, K: int, lda: int, ldb: int, ldc: int,
                 precision: int = PRECISION_3XTF32, stream=None) -> None:
    """``C = A @ B`` column-sharded over the ranks of ``comm``; every rank ends with all of C."""
    rc = load().b200_gemm_f32_sharded(comm._h, mode, _ptr(A), _ptr(B), _ptr(C), M, N, K, lda, ldb, ldc, precision,
                                      _stream_ptr(stream))
    _check(rc, "b200_gemm_f32_sharded")


def matmul_host_sharded(comm: ShardComm, a_rows, b_cols, c_cols, *, M: int, N: int, K: int, chunks: int = 0) -> None:
    """The sharded product from host buffers (numpy float32 arrays: this rank's rows of A, its columns
    of B, its columns of C); returns when the result is on the host."""
    rc = load().b200_matmul_f32_host_sharded(comm._h, a_rows.ctypes.data, b_cols.ctypes.data, c_cols.ctypes.data,
                                             M, N, K, chunks)
    _check(rc, "b200_matmul_f32_host_sharded")


def status() -> None:
    """Synchronises the current device and raises if a bounded device-side wait ran out."""
    _check(load().b200_gemm_status(), "b200_gemm_status")


def selftest_timeout(budget_us: int = 1000):
    """Makes one bounded device-side wait run out on purpose (nothing faults).  Returns
    ``(threads_that_wrongly_completed, abort_flag)``; :func:`status` raises once afterwards."""
    seen = (ctypes.c_int * 2)(-1, -1)
    _check(load().b200_gemm_selftest_timeout(int(budget_us), seen), "b200_gemm_selftest_timeout")
    return int(seen[0]), int(seen[1])


def launch_count() -> int:
    return int(load().b200_gemm_launch_count())


def set_option(name: str, value: int) -> None:
    _check(load().b200_gemm_set_option(name.encode(), int(value)), f"b200_gemm_set_option({name})")
