"""Shared fixtures.  Tests that need a B200 are marked ``gpu``; everything else runs on CPU."""
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100)")


@pytest.fixture(scope="session")
def pkg():
    import __graft_entry__ as entry

    return entry.load_package()


@pytest.fixture(scope="session")
def orc():
    from oracle import oracle_py

    oracle_py.oracle()
    return oracle_py


@pytest.fixture(scope="session")
def golden_dir():
    return ROOT / "tests" / "golden"


@pytest.fixture(scope="session")
def cuda(pkg):
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.cuda.set_device(0)
    pkg.load()
    return torch.device("cuda", 0)
