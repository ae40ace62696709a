"""Host-side mirror of the reference engine's matrix-product interface.

Same names, argument meaning and error behaviour as the reference's ``Tensor::matmul``
(src/tensor_ops.cpp:475-588) and its device seam ``cuda::ops::matmul``
(include/engine/detail/cuda_ops.hpp:46-47), so parity tests read like the reference's own.
Storage is a contiguous float32 torch CUDA tensor; every product runs in the sm_100a library
through its C ABI.  The backward pass calls the transposed forms directly (``dA = dC x B^T``
as an NT product, ``dB = A^T x dC`` as a TN product) instead of materialising transposes the
way the reference does (src/tensor_ops.cpp:576, :581); the values are the same products.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

from . import lib as _lib

_ws_cache = {}


def _workspace(device, nbytes: int):
    """Grow-only scratch per device for the split-K path (the reference keeps one scratch
    buffer the same way, src/cuda/kernels.cu:593-604)."""
    import torch

    if nbytes <= 0:
        return None, 0
    key = (device.type, device.index)
    buf = _ws_cache.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _ws_cache[key] = buf
    return buf, nbytes


def _check_operand(t, name: str) -> None:
    import torch

    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch tensor")
    if not t.is_cuda:
        raise RuntimeError(f"{name} must live on a CUDA device: there is no CPU path")
    if t.dtype != torch.float32:
        raise TypeError(f"{name} must be float32")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous (row-major, last stride 1)")


def _batch_plan(a_shape: Sequence[int], b_shape: Sequence[int]):
    """The reference's shape rules (src/tensor_ops.cpp:476-503)."""
    if len(a_shape) < 2 or len(b_shape) < 2:
        raise ValueError("MatMul requires at least 2 dimensions in both operands.")
    batch_a, batch_b = list(a_shape[:-2]), list(b_shape[:-2])
    a_batched, b_batched = bool(batch_a), bool(batch_b)
    if a_batched and b_batched and batch_a != batch_b:
        raise ValueError(f"Batched MatMul needs identical batch axes: {tuple(a_shape)} and {tuple(b_shape)}.")
    batch_dims = batch_a if a_batched else batch_b
    M, K = a_shape[-2], a_shape[-1]
    K2, N = b_shape[-2], b_shape[-1]
    if K != K2:
        raise ValueError(f"Incompatible dimensions for MatMul: {tuple(a_shape)} and {tuple(b_shape)}.")
    batch = 1
    for d in batch_dims:
        batch *= d
    return batch_dims, batch, M, K, N, a_batched, b_batched


def ops_matmul(a, b, out, batch: int, rows: int, inner_dim: int, cols: int, a_batched: bool,
               b_batched: bool, beta: float = 0.0, *, precision: int = _lib.PRECISION_3XTF32,
               stream=None) -> bool:
    """``out = a x b + beta * out`` — the seam ``cuda::ops::matmul``.  Always returns True:
    the device does the work or an exception is raised (the reference returns False to send
    the caller to its CPU loop; there is no such path here)."""
    ws_bytes = _lib.workspace_bytes(batch, rows, cols, inner_dim)
    ws, ws_bytes = _workspace(out.device, ws_bytes)
    _lib.gemm(a, b, out, batch=batch, M=rows, N=cols, K=inner_dim, lda=inner_dim, ldb=cols, ldc=cols,
              strideA=rows * inner_dim if a_batched else 0,
              strideB=inner_dim * cols if b_batched else 0, strideC=rows * cols, beta=beta,
              precision=precision, workspace=ws, workspace_bytes=ws_bytes, stream=stream)
    return True


def matmul(a, b, *, precision: int = _lib.PRECISION_3XTF32, stream=None):
    """``Tensor::matmul`` on raw torch tensors: (B..., M, K) x (B..., K, N) -> (B..., M, N),
    or one 2-D operand shared by every matrix of the other's batch."""
    import torch

    _check_operand(a, "a")
    _check_operand(b, "b")
    batch_dims, batch, M, K, N, a_batched, b_batched = _batch_plan(a.shape, b.shape)
    out = torch.empty(list(batch_dims) + [M, N], dtype=torch.float32, device=a.device)
    if out.numel() == 0:
        return out
    ops_matmul(a, b, out, batch, M, K, N, a_batched, b_batched, 0.0, precision=precision,
               stream=stream)
    return out


def matmul_backward(a, b, grad_out, *, precision: int = _lib.PRECISION_3XTF32, stream=None,
                    need_a: bool = True, need_b: bool = True):
    """Gradients of ``C = a.matmul(b)`` for a given ``dC`` (src/tensor_ops.cpp:570-585).

    ``dA = dC x B^T`` (NT) and ``dB = A^T x dC`` (TN).  The gradient of an operand shared
    across the batch is the sum over the batch: because the shared operand makes the batch
    just more rows of one product, it is computed as ONE product with the batch folded into
    the contraction (dB) or the rows (dA), instead of a batched product followed by a sum.
    """
    import torch

    _check_operand(a, "a")
    _check_operand(b, "b")
    _check_operand(grad_out, "grad_out")
    batch_dims, batch, M, K, N, a_batched, b_batched = _batch_plan(a.shape, b.shape)
    if list(grad_out.shape) != list(batch_dims) + [M, N]:
        raise ValueError(f"Gradient shape {tuple(grad_out.shape)} incompatible with the product's "
                         f"{tuple(list(batch_dims) + [M, N])}.")
    dA = dB = None

    def run(A_, B_, C_, **kw):
        ws_bytes = _lib.workspace_bytes(kw["batch"], kw["M"], kw["N"], kw["K"])
        ws, ws_bytes = _workspace(C_.device, ws_bytes)
        _lib.gemm(A_, B_, C_, precision=precision, workspace=ws, workspace_bytes=ws_bytes,
                  stream=stream, **kw)

    if need_a:
        dA = torch.empty_like(a)
        if a_batched or batch == 1:
            # dA[b] = dC[b] (M x N) x B[b]^T, B stored K x N  -> NT form
            run(grad_out, b, dA, batch=batch, M=M, N=K, K=N, transB=True, lda=N, ldb=N, ldc=K,
                strideA=M * N, strideB=K * N if b_batched else 0, strideC=M * K)
        else:
            # A is shared, B batched: dA = sum_b dC[b] x B[b]^T = [dC_0 | dC_1 | ...] x [B_0 | B_1 | ...]^T.
            # With row-major storage that is a batched product summed by beta = 1 accumulation
            # in ascending batch order.
            for bi in range(batch):
                run(grad_out[bi] if grad_out.dim() > 2 else grad_out, b[bi], dA, batch=1, M=M, N=K,
                    K=N, transB=True, lda=N, ldb=N, ldc=K, beta=0.0 if bi == 0 else 1.0)
    if need_b:
        dB = torch.empty_like(b)
        if b_batched or batch == 1:
            # dB[b] = A[b]^T (A stored M x K) x dC[b]  -> TN form
            run(a, grad_out, dB, batch=batch, M=K, N=N, K=M, transA=True, lda=K, ldb=N, ldc=N,
                strideA=M * K if a_batched else 0, strideB=M * N, strideC=K * N)
        else:
            # B is shared, A batched: A is (batch*M) x K and dC is (batch*M) x N, both
            # contiguous, so dB = A_flat^T x dC_flat is one TN product over batch*M rows.
            run(a, grad_out, dB, batch=1, M=K, N=N, K=batch * M, transA=True, lda=K, ldb=N, ldc=N)
    return dA, dB


def linear(x, weight, bias=None, *, relu: bool = False, precision: int = _lib.PRECISION_3XTF32, stream=None):
    """``Linear::forward`` (src/nn.cpp:101-130): leading axes flattened, ``flat.matmul(weight)`` with the
    weight stored (in, out), bias broadcast over rows — and, fused into the same kernel's store, the
    bias add and an optional ReLU (the feed-forward ``ff1(x).relu()``, src/transformer.cpp:413)."""
    import torch

    _check_operand(x, "x")
    _check_operand(weight, "weight")
    if weight.dim() != 2 or x.shape[-1] != weight.shape[0]:
        raise ValueError(f"Linear expects (..., {weight.shape[0]}) inputs, got {tuple(x.shape)}.")
    if bias is not None:
        _check_operand(bias, "bias")
        if list(bias.shape) != [weight.shape[1]]:
            raise ValueError("bias must have one value per output feature")
    rows = x.numel() // x.shape[-1]
    K, N = weight.shape
    out = torch.empty(list(x.shape[:-1]) + [N], dtype=torch.float32, device=x.device)
    if out.numel() == 0:
        return out
    ws_bytes = _lib.workspace_bytes(1, rows, N, K)
    ws, ws_bytes = _workspace(x.device, ws_bytes)
    _lib.gemm_fused(x, weight, out, batch=1, M=rows, N=N, K=K, lda=K, ldb=N, ldc=N, bias=bias, relu=relu,
                    precision=precision, workspace=ws, workspace_bytes=ws_bytes, stream=stream)
    return out


def attention_scores(q, k, scale: float, mask=None, *, precision: int = _lib.PRECISION_3XTF32, stream=None):
    """``scores = q.matmul(k.transpose()) * scale + mask`` (src/transformer.cpp:292-297) as ONE kernel:
    K is read as stored (transB), the scale is the product's alpha and the additive mask, shared by
    every head, is added in the store.  q, k: (..., S, d); mask: (S, S) or None."""
    import torch

    _check_operand(q, "q")
    _check_operand(k, "k")
    if q.dim() < 2 or list(q.shape[:-2]) != list(k.shape[:-2]) or q.shape[-1] != k.shape[-1]:
        raise ValueError(f"attention needs matching batch axes and head size: {tuple(q.shape)} and {tuple(k.shape)}.")
    S, d, Sk = q.shape[-2], q.shape[-1], k.shape[-2]
    batch = q.numel() // (S * d) if S * d else 0
    if mask is not None:
        _check_operand(mask, "mask")
        if list(mask.shape) != [S, Sk]:
            raise ValueError("mask must be (S_q, S_k)")
    out = torch.empty(list(q.shape[:-2]) + [S, Sk], dtype=torch.float32, device=q.device)
    if out.numel() == 0:
        return out
    _lib.gemm_fused(q, k, out, batch=batch, M=S, N=Sk, K=d, transB=True, lda=d, ldb=d, ldc=Sk,
                    strideA=S * d, strideB=Sk * d, strideC=S * Sk, alpha=float(scale), addend=mask,
                    ld_addend=Sk, precision=precision, stream=stream)
    return out


def _attention_workspace(device, *, batch, heads, s_q, s_k, d_k, d_v, backward, have_weights=False):
    """Scratch for heads the fused attention kernels do not take (0 bytes when they do; the forward
    uses the caller's weights buffer when there is one)."""
    import torch

    nbytes = _lib.attention_any_workspace(batch=batch, heads=heads, s_q=s_q, s_k=s_k, d_k=d_k, d_v=d_v,
                                          backward=backward)
    if nbytes == 0 or (have_weights and not backward):
        return None, 0
    return torch.empty(nbytes, dtype=torch.uint8, device=device), nbytes


def scaled_dot_product_attention(query, key, value, mask=None, *, return_weights: bool = False,
                                 precision: int = _lib.PRECISION_3XTF32, stream=None):
    """``scaled_dot_product_attention`` (src/transformer.cpp:279-304): softmax(Q K^T / sqrt(d_k) + mask) V
    over the leading (batch, head) axes, fused into one kernel; the (.., S, S) scores never reach global
    memory.  Returns ``out`` or ``(out, attention_weights)``."""
    import math

    import torch

    for name, t in (("query", query), ("key", key), ("value", value)):
        _check_operand(t, name)
        if t.dim() < 2:
            raise ValueError("Attention needs at least 2 dimensions (seq, d_k).")
    d_k = query.shape[-1]
    if key.shape[-1] != d_k:
        raise ValueError(f"Query and key must share d_k: {tuple(query.shape)} and {tuple(key.shape)}.")
    lead = list(query.shape[:-2])
    if list(key.shape[:-2]) != lead or list(value.shape[:-2]) != lead or key.shape[-2] != value.shape[-2]:
        raise ValueError("query, key and value need the same leading axes and key/value the same length")
    s_q, s_k, d_v = query.shape[-2], key.shape[-2], value.shape[-1]
    if mask is not None:
        _check_operand(mask, "mask")
        if list(mask.shape) != [s_q, s_k]:
            raise ValueError("mask must be (S_q, S_k)")
    batch = 1
    for d in lead:
        batch *= d
    out = torch.empty(lead + [s_q, d_v], dtype=torch.float32, device=query.device)
    weights = torch.empty(lead + [s_q, s_k], dtype=torch.float32, device=query.device) if return_weights else None
    if batch:
        ws, ws_bytes = _attention_workspace(query.device, batch=batch, heads=1, s_q=s_q, s_k=s_k, d_k=d_k, d_v=d_v,
                                            backward=False, have_weights=weights is not None)
        _lib.attention_any(query, key, value, mask, out, weights, batch=batch, heads=1, s_q=s_q, s_k=s_k, d_k=d_k,
                           d_v=d_v, q_strides=(s_q * d_k, 0, d_k), k_strides=(s_k * d_k, 0, d_k),
                           v_strides=(s_k * d_v, 0, d_v), out_strides=(s_q * d_v, 0, d_v),
                           scale=1.0 / math.sqrt(float(d_k)), precision=precision, workspace=ws,
                           workspace_bytes=ws_bytes, stream=stream)
    return (out, weights) if return_weights else out


def scaled_dot_product_attention_backward(query, key, value, grad_out, mask=None, *,
                                          precision: int = _lib.PRECISION_3XTF32, stream=None):
    """The gradients autograd hands query, key and value of ``scaled_dot_product_attention`` for ``grad_out``
    (the backward of the five nodes of src/transformer.cpp:279-304), as ONE kernel that recomputes the
    attention weights: ``(grad_query, grad_key, grad_value)``.  Heads whose tiles do not fit one CTA
    (S = 64 with head widths up to 64 do) run composed on the device: four batched products through the
    transposed forms and one row kernel for the softmax backward."""
    import math

    import torch

    for name, t in (("query", query), ("key", key), ("value", value), ("grad_out", grad_out)):
        _check_operand(t, name)
        if t.dim() < 2:
            raise ValueError("Attention needs at least 2 dimensions (seq, d_k).")
    d_k = query.shape[-1]
    if key.shape[-1] != d_k:
        raise ValueError(f"Query and key must share d_k: {tuple(query.shape)} and {tuple(key.shape)}.")
    lead = list(query.shape[:-2])
    if list(key.shape[:-2]) != lead or list(value.shape[:-2]) != lead or key.shape[-2] != value.shape[-2]:
        raise ValueError("query, key and value need the same leading axes and key/value the same length")
    s_q, s_k, d_v = query.shape[-2], key.shape[-2], value.shape[-1]
    if list(grad_out.shape) != lead + [s_q, d_v]:
        raise ValueError(f"grad_out must be {tuple(lead + [s_q, d_v])}, received {tuple(grad_out.shape)}.")
    if mask is not None:
        _check_operand(mask, "mask")
        if list(mask.shape) != [s_q, s_k]:
            raise ValueError("mask must be (S_q, S_k)")
    batch = 1
    for d in lead:
        batch *= d
    gq, gk, gv = torch.empty_like(query), torch.empty_like(key), torch.empty_like(value)
    if batch:
        ws, ws_bytes = _attention_workspace(query.device, batch=batch, heads=1, s_q=s_q, s_k=s_k, d_k=d_k, d_v=d_v,
                                            backward=True)
        _lib.attention_backward_any(
            query, key, value, mask, grad_out, gq, gk, gv, batch=batch, heads=1, s_q=s_q, s_k=s_k, d_k=d_k, d_v=d_v,
            q_strides=(s_q * d_k, 0, d_k), k_strides=(s_k * d_k, 0, d_k), v_strides=(s_k * d_v, 0, d_v),
            out_strides=(s_q * d_v, 0, d_v), scale=1.0 / math.sqrt(float(d_k)), precision=precision, workspace=ws,
            workspace_bytes=ws_bytes, stream=stream)
    return gq, gk, gv


def multi_head_attention_core_backward(query, key, value, grad_merged, num_heads: int, mask=None, *,
                                       precision: int = _lib.PRECISION_3XTF32, stream=None):
    """Backward of ``multi_head_attention_core``: from the gradient of the merged context (B, S, d_model) to the
    gradients of the three projections (B, S, d_model), heads addressed by strides both ways."""
    import math

    import torch

    for name, t in (("query", query), ("key", key), ("value", value), ("grad_merged", grad_merged)):
        if not isinstance(t, torch.Tensor) or not t.is_cuda or t.dtype != torch.float32:
            raise TypeError(f"{name} must be a float32 CUDA tensor")
        if t.dim() != 3 or t.stride(2) != 1:
            raise ValueError(f"{name} must be (batch, seq, d_model), dense along its last axis")
    batch, s_q, d_model = query.shape
    s_k = key.shape[1]
    if num_heads <= 0 or d_model % num_heads != 0 or value.shape[2] % num_heads != 0:
        raise ValueError("d_model must be divisible by num_heads.")
    d_k, d_v = d_model // num_heads, value.shape[2] // num_heads
    if list(grad_merged.shape) != [batch, s_q, num_heads * d_v]:
        raise ValueError("grad_merged must have the shape of the merged context")
    if mask is not None:
        _check_operand(mask, "mask")
    # gradients in the projections' own layout (also when those are column slices of one tensor)
    gq, gk, gv = (torch.empty_strided(t.shape, t.stride(), dtype=torch.float32, device=t.device)
                  for t in (query, key, value))
    if batch:
        ws, ws_bytes = _attention_workspace(query.device, batch=batch, heads=num_heads, s_q=s_q, s_k=s_k, d_k=d_k,
                                            d_v=d_v, backward=True)
        _lib.attention_backward_any(
            query, key, value, mask, grad_merged, gq, gk, gv, batch=batch, heads=num_heads, s_q=s_q, s_k=s_k, d_k=d_k,
            d_v=d_v, q_strides=(query.stride(0), d_k, query.stride(1)), k_strides=(key.stride(0), d_k, key.stride(1)),
            v_strides=(value.stride(0), d_v, value.stride(1)),
            out_strides=(grad_merged.stride(0), d_v, grad_merged.stride(1)), scale=1.0 / math.sqrt(float(d_k)),
            precision=precision, workspace=ws, workspace_bytes=ws_bytes, stream=stream)
    return gq, gk, gv


def multi_head_attention_core(query, key, value, num_heads: int, mask=None, *, return_weights: bool = False,
                              precision: int = _lib.PRECISION_3XTF32, stream=None):
    """The middle of ``MultiHeadAttention::forward`` (src/transformer.cpp:339-357): from the three projections
    (B, S, d_model) to the merged context (B, S, d_model).  The reference materialises
    ``reshape(B, S, H, hd).permute(0, 2, 1, 3)`` three times and the inverse permute once; here the fused
    attention kernel reads each head through strides and writes the merged layout directly.  The projections
    may be column slices of one wider tensor (a fused Q|K|V product): only the last axis must be dense.
    Returns ``merged`` or ``(merged, attention_weights)`` with the weights shaped (B, H, S_q, S_k)."""
    import math

    import torch

    for name, t in (("query", query), ("key", key), ("value", value)):
        if not isinstance(t, torch.Tensor):
            raise TypeError(f"{name} must be a torch tensor")
        if not t.is_cuda:
            raise RuntimeError(f"{name} must live on a CUDA device: there is no CPU path")
        if t.dtype != torch.float32:
            raise TypeError(f"{name} must be float32")
        if t.dim() != 3:
            raise ValueError(f"MultiHeadAttention expects (batch, seq, d_model), received {tuple(t.shape)}.")
        if t.stride(2) != 1:
            raise ValueError(f"{name} must be dense along its last axis")
    if num_heads <= 0 or query.shape[2] % num_heads != 0 or value.shape[2] % num_heads != 0:
        raise ValueError("d_model must be divisible by num_heads.")
    batch, s_q, d_model = query.shape
    if key.shape[0] != batch or value.shape[0] != batch or key.shape[2] != d_model or key.shape[1] != value.shape[1]:
        raise ValueError("query, key and value need the same batch, key/value the same length and query/key the "
                         "same width")
    s_k = key.shape[1]
    d_k, d_v = d_model // num_heads, value.shape[2] // num_heads
    if mask is not None:
        _check_operand(mask, "mask")
        if list(mask.shape) != [s_q, s_k]:
            raise ValueError("mask must be (S_q, S_k)")
    out = torch.empty((batch, s_q, num_heads * d_v), dtype=torch.float32, device=query.device)
    weights = (torch.empty((batch, num_heads, s_q, s_k), dtype=torch.float32, device=query.device)
               if return_weights else None)
    if batch:
        ws, ws_bytes = _attention_workspace(query.device, batch=batch, heads=num_heads, s_q=s_q, s_k=s_k, d_k=d_k,
                                            d_v=d_v, backward=False, have_weights=weights is not None)
        _lib.attention_any(
            query, key, value, mask, out, weights, batch=batch, heads=num_heads, s_q=s_q, s_k=s_k, d_k=d_k, d_v=d_v,
            q_strides=(query.stride(0), d_k, query.stride(1)), k_strides=(key.stride(0), d_k, key.stride(1)),
            v_strides=(value.stride(0), d_v, value.stride(1)), out_strides=(out.stride(0), d_v, out.stride(1)),
            scale=1.0 / math.sqrt(float(d_k)), precision=precision, workspace=ws, workspace_bytes=ws_bytes,
            stream=stream)
    return (out, weights) if return_weights else out


def conv2d(x, weight, bias=None, *, stride: int = 1, padding: int = 0, relu: bool = False,
           precision: int = _lib.PRECISION_3XTF32, stream=None):
    """``Conv2d::forward`` (src/conv.cpp:280-338): x (N, C, H, W), weight (outC, C, kH, kW), optional bias
    (outC,) -> (N, outC, oH, oW).  One implicit-GEMM kernel instead of im2col + product + bias + permute."""
    import torch

    _check_operand(x, "x")
    _check_operand(weight, "weight")
    if x.dim() != 4:
        raise ValueError(f"Conv2d expects a 4D volume (N, C, H, W), received {tuple(x.shape)}.")
    if weight.dim() != 4 or x.shape[1] != weight.shape[1]:
        raise ValueError(f"Conv2d with in_channels={weight.shape[1] if weight.dim() == 4 else '?'} "
                         f"received an input {tuple(x.shape)}.")
    if stride < 1 or padding < 0:
        raise ValueError("Conv2d requires a stride greater than zero and a non-negative padding.")
    n, c, h, w = x.shape
    out_c, _, kh, kw = weight.shape
    if bias is not None:
        _check_operand(bias, "bias")
        if list(bias.shape) != [out_c]:
            raise ValueError("bias must have one value per output channel")
    if h + 2 * padding < kh or w + 2 * padding < kw:
        raise ValueError("the window does not fit the padded input")
    oh, ow = (h + 2 * padding - kh) // stride + 1, (w + 2 * padding - kw) // stride + 1
    y = torch.empty((n, out_c, oh, ow), dtype=torch.float32, device=x.device)
    if y.numel():
        _lib.conv2d_forward(x, weight, bias, y, n=n, c=c, h=h, w=w, out_c=out_c, kh=kh, kw=kw, stride=stride,
                            pad=padding, relu=relu, precision=precision, stream=stream)
    return y


def conv2d_backward(x, weight, grad_out, *, stride: int = 1, padding: int = 0, need_input_grad: bool = True,
                    need_weight_grad: bool = True, need_bias_grad: bool = True, accumulate_into=None,
                    precision: int = _lib.PRECISION_3XTF32, stream=None):
    """The gradients ``Conv2d`` receives from autograd (src/conv.cpp:280-338 composed with the product's
    backward, src/tensor_ops.cpp:570-585, and im2col's, src/conv.cpp:236-257), for grad_out (N, outC, oH, oW):
    ``(grad_x, grad_weight, grad_bias)``, ``None`` where not needed.  No column matrix, no transposes and no
    col2im scatter are built: one gather kernel per gradient.  ``accumulate_into=(gx, gw, gb)`` adds into
    existing gradients instead (``Tensor::add_grad``); entries may be ``None``."""
    import torch

    _check_operand(x, "x")
    _check_operand(weight, "weight")
    _check_operand(grad_out, "grad_out")
    if x.dim() != 4 or weight.dim() != 4 or x.shape[1] != weight.shape[1]:
        raise ValueError(f"Conv2d gradients need x (N, C, H, W) and weight (outC, C, kH, kW), received "
                         f"{tuple(x.shape)} and {tuple(weight.shape)}.")
    if stride < 1 or padding < 0:
        raise ValueError("Conv2d requires a stride greater than zero and a non-negative padding.")
    n, c, h, w = x.shape
    out_c, _, kh, kw = weight.shape
    if h + 2 * padding < kh or w + 2 * padding < kw:
        raise ValueError("the window does not fit the padded input")
    oh, ow = (h + 2 * padding - kh) // stride + 1, (w + 2 * padding - kw) // stride + 1
    if list(grad_out.shape) != [n, out_c, oh, ow]:
        raise ValueError(f"grad_out must be {(n, out_c, oh, ow)}, received {tuple(grad_out.shape)}.")
    beta = 0.0
    if accumulate_into is not None:
        gx, gw, gb = accumulate_into
        beta = 1.0
        for name, g, ref in (("grad_x", gx, x), ("grad_weight", gw, weight)):
            if g is not None:
                _check_operand(g, name)
                if g.shape != ref.shape:
                    raise ValueError(f"{name} must have the shape of its tensor")
        if gb is not None:
            _check_operand(gb, "grad_bias")
            if list(gb.shape) != [out_c]:
                raise ValueError("grad_bias must have one value per output channel")
    else:
        gx = torch.empty_like(x) if need_input_grad else None
        gw = torch.empty_like(weight) if need_weight_grad else None
        gb = torch.empty((out_c,), dtype=torch.float32, device=x.device) if need_bias_grad else None
    dims = dict(n=n, c=c, h=h, w=w, out_c=out_c, kh=kh, kw=kw, stride=stride, pad=padding)
    ws, ws_bytes = _workspace(x.device, _lib.conv2d_backward_workspace(**dims) if gw is not None else 0)
    _lib.conv2d_backward(x, weight, grad_out, gx, gw, gb, beta=beta, precision=precision, workspace=ws,
                         workspace_bytes=ws_bytes, stream=stream, **dims)
    return gx, gw, gb


class Tensor:
    """The slice of ``engine::Tensor`` the matrix-product path needs: a value, an optional
    gradient, ``matmul`` and ``backward`` (include/engine/tensor.hpp:157-198)."""

    def __init__(self, data, requires_grad: bool = False):
        _check_operand(data, "data")
        self.data = data
        self.requires_grad = requires_grad
        self.grad: Optional["Tensor"] = None
        self._parents: Tuple["Tensor", ...] = ()
        self._backward_fn = None

    @property
    def shape(self) -> List[int]:
        return list(self.data.shape)

    def matmul(self, other: "Tensor") -> "Tensor":
        out = Tensor(matmul(self.data, other.data), self.requires_grad or other.requires_grad)
        if out.requires_grad:
            a, b = self, other
            out._parents = (a, b)

            def backward_fn(grad_out):
                dA, dB = matmul_backward(a.data, b.data, grad_out, need_a=a.requires_grad,
                                         need_b=b.requires_grad)
                if a.requires_grad:
                    a.add_grad(dA)
                if b.requires_grad:
                    b.add_grad(dB)

            out._backward_fn = backward_fn
        return out

    def add_grad(self, g) -> None:
        """First write copies, later writes accumulate (src/tensor.cpp:168-203)."""
        if not self.requires_grad:
            return
        if list(g.shape) != self.shape:
            raise ValueError(f"Gradient shape {tuple(g.shape)} incompatible with the tensor's "
                             f"{tuple(self.shape)}.")
        if self.grad is None:
            self.grad = Tensor(g.clone())
        else:
            self.grad.data += g

    def backward(self, grad_output) -> None:
        """Reverse sweep over the recorded products (src/autograd.cpp:104-156)."""
        order, seen = [], set()
        stack = [(self, False)]
        while stack:
            node, done = stack.pop()
            if done:
                order.append(node)
                continue
            if id(node) in seen:
                continue
            seen.add(id(node))
            stack.append((node, True))
            for parent in node._parents:
                stack.append((parent, False))
        grads = {id(self): grad_output.data if isinstance(grad_output, Tensor) else grad_output}
        self.add_grad(grads[id(self)])
        for node in reversed(order):
            if node._backward_fn is not None and node.grad is not None:
                node._backward_fn(node.grad.data)
