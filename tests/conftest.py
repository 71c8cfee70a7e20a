import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def cuda_lib():
    """The built C-ABI library on a CUDA device; fails (never skips) if it cannot be used."""
    import torch

    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from hackaton_b200 import _lib

    _lib.lib()
    props = _lib.query(0)
    assert props.supported == 1, f"device is sm_{props.cc_major}{props.cc_minor}, need sm_100"
    return _lib
