import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def pkg():
    """The ctypes binding of the product library (built on demand; no fallback)."""
    if not (ROOT / "c-ml_b200" / "lib" / "libcml_b200.so").exists():
        entry.build()
    return entry.load_package()


@pytest.fixture(scope="session")
def synth(pkg):
    return entry.load_synth()


@pytest.fixture(scope="session")
def ob():
    return entry.load_oracle_binding()


@pytest.fixture(scope="session")
def orc(ob):
    return ob.load_orc()


@pytest.fixture(scope="session")
def ref(ob):
    """The compiled C-ML reference, or None where oracle/_ref/ was not built."""
    return ob.load_ref()


@pytest.fixture(scope="session")
def golden():
    return np.load(ROOT / "tests" / "golden" / "golden.npz")


@pytest.fixture(scope="session")
def torch_dev():
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    return torch.device("cuda:0")


def rel_err(got, want, floor=1e-3):
    """max_i |got-want| / max(|want_i|, floor * max|want|): element-wise relative error with
    a floor so that near-zero outputs do not divide by nothing."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    scale = np.maximum(np.abs(want), floor * np.abs(want).max())
    return float((np.abs(got - want) / scale).max())


def rel_err_inf(got, want):
    """||got-want||_inf / ||want||_inf."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    return float(np.abs(got - want).max() / np.abs(want).max())
