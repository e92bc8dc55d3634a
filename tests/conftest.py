"""pytest configuration: the `gpu` marker, and one-time builds of the checker and the library."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def _has_gpu():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session", autouse=True)
def _built():
    """Build the CPU checker (oracle/) and, if it is not there yet, the CUDA library."""
    oracle_dir = os.path.join(ROOT, "oracle")
    if not os.path.exists(os.path.join(oracle_dir, "liboracle.so")):
        subprocess.run(["make", "-C", oracle_dir], check=True, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    from fp8_quant_matmul_b200 import build
    build.build_all()
    yield
