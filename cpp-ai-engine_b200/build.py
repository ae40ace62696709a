"""Builds ``libb200gemm.so`` in-tree with nvcc for sm_100a (cross-compiles without a GPU)."""
from __future__ import annotations

import os
import shutil
import subprocess
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB = PKG_DIR / "libb200gemm.so"
SOURCES = [CSRC / "gemm_sm100.cu", CSRC / "shard_sm100.cu", CSRC / "attention_any.cu"]
HEADERS = [CSRC / "gemm_kernel.cuh", CSRC / "attention_kernel.cuh", CSRC / "attention_bwd_kernel.cuh", CSRC / "sm100_ptx.cuh", CSRC / "shard_layout.h", PKG_DIR.parent / "include" / "b200_gemm.h"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
    "-cudart", "static",
    "-ldl",  # NCCL is resolved at run time (dlopen), never linked
]


def nvcc_path() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found: set NVCC or put it on PATH")
    return cand


def is_stale() -> bool:
    if not LIB.exists():
        return True
    built = LIB.stat().st_mtime
    return any(f.stat().st_mtime > built for f in SOURCES + HEADERS)


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compiles the CUDA sources into ``libb200gemm.so`` next to this file."""
    if not force and not is_stale():
        return LIB
    cmd = [nvcc_path(), *NVCC_FLAGS]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", str(LIB), *map(str, SOURCES)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + proc.stdout + proc.stderr)
    if verbose:
        print(proc.stderr)
    return LIB


HOST_DIR = PKG_DIR / "host"
HOST_LIB = PKG_DIR / "libengine_b200.so"
CUDA_HOME = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))


def cxx_path() -> str:
    return os.environ.get("CXX") or shutil.which("g++") or "g++"


def build_host_library(force: bool = False) -> Path:
    """Compiles the C++17 host side (engine::Tensor / Storage / cuda::ops::matmul over the C ABI)
    into ``libengine_b200.so`` next to the CUDA library."""
    src = HOST_DIR / "engine_b200.cpp"
    deps = [src, HOST_DIR / "engine_b200.hpp", PKG_DIR.parent / "include" / "b200_gemm.h"]
    if not force and HOST_LIB.exists() and all(d.stat().st_mtime <= HOST_LIB.stat().st_mtime for d in deps):
        return HOST_LIB
    build_library()
    cmd = [cxx_path(), "-std=c++17", "-O2", "-Wall", "-Wextra", "-fPIC", "-shared",
           "-I", str(PKG_DIR.parent / "include"), "-I", str(CUDA_HOME / "include"), str(src),
           "-o", str(HOST_LIB), "-L", str(PKG_DIR), "-lb200gemm", "-L", str(CUDA_HOME / "lib64"), "-lcudart",
           "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{CUDA_HOME / 'lib64'}"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("host library build failed:\n" + proc.stdout + proc.stderr)
    return HOST_LIB


def build_host_tests(force: bool = False) -> Path:
    """Compiles tests/cpp/test_engine_b200 (links the host library and, as its checker, the oracle)."""
    root = PKG_DIR.parent
    src = root / "tests" / "cpp" / "test_engine_b200.cpp"
    exe = root / "tests" / "cpp" / "test_engine_b200"
    build_host_library(force)
    if not force and exe.exists() and exe.stat().st_mtime >= max(src.stat().st_mtime, HOST_LIB.stat().st_mtime):
        return exe
    cmd = [cxx_path(), "-std=c++17", "-O2", "-Wall", "-Wextra", str(src), "-I", str(HOST_DIR),
           "-I", str(root / "include"), "-o", str(exe), "-L", str(PKG_DIR), "-lengine_b200", "-lb200gemm",
           "-L", str(root / "oracle"), "-loracle", "-L", str(CUDA_HOME / "lib64"), "-lcudart",
           "-Wl,-rpath,$ORIGIN/../../cpp-ai-engine_b200", "-Wl,-rpath,$ORIGIN/../../oracle",
           f"-Wl,-rpath,{CUDA_HOME / 'lib64'}", "-lpthread"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("host test build failed:\n" + proc.stdout + proc.stderr)
    return exe


def build_shard_test(force: bool = False) -> Path:
    """Compiles tests/cpp/test_shard_b200 (a C++ caller of the sharded product on two GPUs; links the
    CUDA library and, as its checker, the oracle; NCCL is found at run time)."""
    root = PKG_DIR.parent
    src = root / "tests" / "cpp" / "test_shard_b200.cpp"
    exe = root / "tests" / "cpp" / "test_shard_b200"
    build_library()
    if not force and exe.exists() and exe.stat().st_mtime >= max(src.stat().st_mtime, LIB.stat().st_mtime):
        return exe
    cmd = [cxx_path(), "-std=c++17", "-O2", "-Wall", "-Wextra", str(src), "-I", str(root / "include"),
           "-I", str(CUDA_HOME / "include"), "-o", str(exe), "-L", str(PKG_DIR), "-lb200gemm",
           "-L", str(root / "oracle"), "-loracle", "-L", str(CUDA_HOME / "lib64"), "-lcudart", "-ldl",
           "-Wl,-rpath,$ORIGIN/../../cpp-ai-engine_b200", "-Wl,-rpath,$ORIGIN/../../oracle",
           f"-Wl,-rpath,{CUDA_HOME / 'lib64'}", "-lpthread"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("shard test build failed:\n" + proc.stdout + proc.stderr)
    return exe
