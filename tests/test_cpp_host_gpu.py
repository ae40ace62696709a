"""Runs the C++17 host-side test program (tests/cpp/test_engine_b200.cpp) on the GPU: the
engine-shaped Tensor / Storage / cuda::ops::matmul surface over the C ABI."""
import subprocess
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def test_cpp_host_suite(cuda):
    exe = ROOT / "tests" / "cpp" / "test_engine_b200"
    if not exe.exists():
        import __graft_entry__ as entry

        entry.build()
    proc = subprocess.run([str(exe), str(ROOT / "tests" / "golden")], capture_output=True, text=True, timeout=600)
    print(proc.stdout[-4000:])
    print(proc.stderr[-2000:])
    assert proc.returncode == 0, proc.stdout[-3000:]
    assert "ALL TESTS PASSED" in proc.stdout
