import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def golden_cpu():
    import numpy as np
    return np.load(os.path.join(ROOT, "tests", "golden", "ref_cpu.npz"))


@pytest.fixture(params=["general", "fused"])
def topk_path(request, monkeypatch):
    """Run a top-k test twice: through the general kernels only (``EKV_FUSED_SMALL=0``) and with the
    one-launch small-problem kernel allowed to take the step when the problem fits it."""
    monkeypatch.setenv("EKV_FUSED_SMALL", "0" if request.param == "general" else "1")
    return request.param
