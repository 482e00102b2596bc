import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session", autouse=True)
def _native_libs():
    """Build the host bookkeeping library and the C oracle if they are missing (both are plain gcc/g++).
    The CUDA library is built by `python -m kriya_rt_b200.build` / `__graft_entry__.build()`."""
    from kriya_rt_b200 import build as B

    B.build_kv()
    from oracle import c_oracle

    c_oracle.build()
    yield


def has_gpu() -> bool:
    try:
        import torch

        return torch.cuda.is_available()
    except Exception:
        return False
