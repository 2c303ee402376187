import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")
    # The shared library, the runner and the oracle are build products (not in the repository):
    # compile whatever is missing or older than its sources before any test imports them.
    from sparsewave_b200 import build as lib_build
    lib_build.build()
    from oracle import build as oracle_build
    oracle_build.build_oracle()
    oracle_build.build_reference()


@pytest.fixture(scope="session")
def ctx():
    """One library context on cuda:0 for the GPU tests."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from sparsewave_b200 import Context
    c = Context(0)
    yield c
    c.close()
