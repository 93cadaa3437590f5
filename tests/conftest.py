import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def abi():
    """C-ABI caller; a GPU test that cannot load the CUDA library must fail, not skip."""
    import torch
    assert torch.cuda.is_available(), "gpu-marked test started without a CUDA device"
    from helpers import Abi
    return Abi()


@pytest.fixture(scope="session")
def ref():
    """The reference's own CUDA extension (prebuilt by oracle/build_ref.py into oracle/_ref/)."""
    from oracle import build_ref
    r = build_ref.load_ref()
    if r is None:
        pytest.skip("oracle/_ref is not built (needs the reference sources at build time)")
    return r
