"""B200-native fp32 GEMM behind the cpp-ai-engine ``Tensor::matmul`` seam.

The product is the C-ABI shared library ``libb200gemm.so`` (CUDA for sm_100a, sources in
``csrc/``, declarations in ``include/b200_gemm.h``).  This package is the thin Python host
side: it builds and loads the library and mirrors the reference's operator interface for
the path (``matmul`` with the engine's batch rules, the two backward forms, and the device
seam ``cuda::ops::matmul``), using torch only for device memory and streams.

There is no CPU fallback: if the library is missing or no sm_100 device is present, calls
raise.
"""
from __future__ import annotations

from . import build as _build  # noqa: F401
from .lib import (  # noqa: F401
    B200Error,
    attention_any,
    attention_any_workspace,
    attention_backward_any,
    attention_forward,
    conv2d_forward,
    PRECISION_3XTF32,
    PRECISION_TF32,
    gemm,
    gemm_colshard,
    gemm_fused,
    gemm_sharded,
    matmul_host_sharded,
    ShardComm,
    SHARD_FUSED,
    SHARD_NCCL,
    shard_columns,
    shard_host_plan,
    gemm_static_scratch,
    launch_count,
    lib_path,
    load,
    matmul_host,
    plan,
    selftest_timeout,
    set_option,
    status,
    workspace_bytes,
)
from . import engine, lib, shard  # noqa: F401
from .engine import Tensor, attention_scores, conv2d, conv2d_backward, linear, multi_head_attention_core, multi_head_attention_core_backward, scaled_dot_product_attention, scaled_dot_product_attention_backward, matmul, matmul_backward, ops_matmul  # noqa: F401
