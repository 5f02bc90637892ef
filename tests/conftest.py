import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "apathy-atlas_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def _ensure_built():
    lib = os.path.join(PKG, "lib", "libatlas_b200.so")
    if not os.path.exists(lib):
        subprocess.run(["make", "-C", PKG, "--no-print-directory"], check=True)
    orc = os.path.join(ROOT, "oracle", "libatlas_oracle.so")
    if not os.path.exists(orc):
        subprocess.run(["make", "-C", os.path.join(ROOT, "oracle"), "--no-print-directory"], check=True)


_ensure_built()


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle_ctypes
    return oracle_ctypes


@pytest.fixture(scope="session")
def atlas():
    import atlas_b200
    atlas_b200.lib()
    return atlas_b200


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    torch.cuda.set_device(0)
    return torch
