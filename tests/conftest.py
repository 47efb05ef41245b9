import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100); run with -m gpu on a B200")


@pytest.fixture(scope="session")
def golden():
    return np.load(ROOT / "tests" / "golden" / "reference_x86_avx2.npz")


@pytest.fixture(scope="session")
def port():
    import oracle
    return oracle.port()


@pytest.fixture(scope="session")
def reference():
    """The reference's own CPU family, when oracle/_ref holds it (or the reference tree is mounted); else None."""
    import oracle
    return oracle.reference()


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran where torch sees no CUDA device")
    torch.cuda.set_device(0)
    return torch


@pytest.fixture(scope="session")
def fam(cuda):
    import silvann_b200
    f = silvann_b200.family()
    assert f.sys.device_count() >= 1
    assert f.sys.bind_device(0) == 1
    return f
