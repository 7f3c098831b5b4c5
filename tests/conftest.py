import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
os.environ.setdefault("MASTER_ADDR", "127.0.0.1")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    return np.load(ROOT / "tests" / "golden" / "reference_ops.npz")


@pytest.fixture(scope="session")
def golden_cfg():
    """Fixtures for the operators the reference lacks, computed through the reference's own multiply and
    fp32 matmul operators (tests/golden/make_golden.py, second half)."""
    import numpy as np
    return np.load(ROOT / "tests" / "golden" / "baseline_configs.npz")


@pytest.fixture(scope="session")
def cuda_device():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from tilebench_b200 import native
    native.require_b200()          # raises (fails the test) if the extension is missing or not sm_100
    return torch.device("cuda:0")
