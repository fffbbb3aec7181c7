import importlib
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def pkg():
    """The product package (its directory name has a hyphen, hence importlib)."""
    return importlib.import_module("dcu-video-dit-turbo_b200")


@pytest.fixture(scope="session")
def ref():
    """The CPU oracle: only tests may use it."""
    from oracle import ref_ops
    return ref_ops


@pytest.fixture(scope="session")
def oracle_c():
    import ctypes
    from oracle import build as oracle_build
    lib = ctypes.CDLL(str(oracle_build.build()))
    lib.oc_recip_mismatches.restype = ctypes.c_int64
    return lib


@pytest.fixture(scope="session")
def cuda_pkg(pkg):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    pkg._lib.load()
    return pkg
